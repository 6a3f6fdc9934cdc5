"""Runs one operator case a few times so a profiler can capture it:

    python -m cudaop_b200.profile_case --case fp8 --size 8192 --iters 3
    ncu --set full --clock-control none -k regex:gemm_fp8 -c 3 -o prof python -m cudaop_b200.profile_case --case fp8

Cases: fp8, swiglu (MLP gate/up shape), rowcol (MLP down shape), nvfp4, sparse, w4a16 (M via --m), quant.
Operands are random bytes of the right formats; nothing is checked here (the parity tests do that).
"""
from __future__ import annotations

import argparse

import torch

import cudaop_b200 as ops


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--m", type=int, default=16)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--nvfp4-pair", type=int, default=-1, help="1/0: force the CTA-pair / one-CTA NVFP4 kernel")
    ap.add_argument("--w4a16-impl", type=int, default=-1, help="b200q_w4a16_set_impl value for the w4a16 case")
    a = ap.parse_args()
    L = ops.lib()
    if a.nvfp4_pair >= 0:
        L.b200q_nvfp4_set_2cta(a.nvfp4_pair)
    if a.w4a16_impl >= 0:
        L.b200q_w4a16_set_impl(a.w4a16_impl)
    st = torch.cuda.current_stream().cuda_stream
    S = a.size
    u8 = lambda *shape, hi=120: torch.randint(0, hi, shape, dtype=torch.uint8, device="cuda")
    if a.case == "fp8":
        A, B = u8(S, S), u8(S, S); C = torch.empty((S, S), dtype=torch.bfloat16, device="cuda")
        fn = lambda i: L.b200q_gemm_fp8(A.data_ptr(), B.data_ptr(), C.data_ptr(), S, S, S, 1.0, 1.0, st)
    elif a.case == "swiglu":
        T, H, I = 4096, 8192, 28672 * S // 8192
        X, Wg, Wu = u8(T, H), u8(I, H), u8(I, H)
        rs, sg, su = (torch.rand(n, device="cuda") for n in (T, I, I))
        Hh = torch.empty((T, I), dtype=torch.bfloat16, device="cuda")
        fn = lambda i: L.b200q_gemm_fp8_swiglu(X.data_ptr(), Wg.data_ptr(), Wu.data_ptr(), Hh.data_ptr(), T, I, H,
                                               rs.data_ptr(), sg.data_ptr(), su.data_ptr(), st)
    elif a.case == "rowcol":
        T, H, I = 4096, 8192, 28672 * S // 8192
        X, W = u8(T, I), u8(H, I)
        rs, cs = torch.rand(T, device="cuda"), torch.rand(H, device="cuda")
        Y = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
        fn = lambda i: L.b200q_gemm_fp8_rowcol(X.data_ptr(), W.data_ptr(), Y.data_ptr(), T, H, I, rs.data_ptr(),
                                               cs.data_ptr(), 0, st)
    elif a.case == "nvfp4":
        A, B = u8(S, S // 2, hi=256), u8(S, S // 2, hi=256)
        sf = torch.randint(0x28, 0x48, (L.b200q_nvfp4_sf_bytes(S, S),), dtype=torch.uint8, device="cuda")
        C = torch.empty((S, S), dtype=torch.bfloat16, device="cuda")
        fn = lambda i: L.b200q_gemm_nvfp4_blocked(A.data_ptr(), sf.data_ptr(), B.data_ptr(), sf.data_ptr(),
                                                  C.data_ptr(), S, S, S, 1.0, 1.0, st)
    elif a.case == "sparse":
        M = S // 2
        A, B = u8(M, S // 2), u8(S, S)
        E = torch.full((M, S // 8), 0xE4, dtype=torch.uint8, device="cuda")
        C = torch.empty((M, S), dtype=torch.bfloat16, device="cuda")
        fn = lambda i: L.b200q_gemm_sp24_fp8(A.data_ptr(), E.data_ptr(), B.data_ptr(), C.data_ptr(), M, S, S, 1.0, 1.0, st)
    elif a.case == "w4a16":
        N = K = 4096; M = a.m; sets = 40      # 40 x 8 MiB of weights: every launch streams from HBM
        W = u8(sets, N, K // 2, hi=256)
        Sc = (torch.rand((sets, N, K // 128), device="cuda") * 0.015 + 0.005).to(torch.float16)
        X = torch.randn((M, K), device="cuda").to(torch.bfloat16)
        Y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        fn = lambda i: L.b200q_gemm_w4a16(X.data_ptr(), W[i % sets].data_ptr(), Sc[i % sets].data_ptr(), Y.data_ptr(),
                                          M, N, K, 128, st)
    elif a.case == "quant":
        T, Cc = 4096, 28672 * S // 8192
        X = torch.randn((T, Cc), device="cuda").to(torch.bfloat16)
        Q = torch.empty((T, Cc), dtype=torch.uint8, device="cuda"); Sx = torch.empty(T, device="cuda")
        fn = lambda i: L.b200q_quant_rows_e4m3(X.data_ptr(), Q.data_ptr(), Sx.data_ptr(), T, Cc, st)
    else:
        raise SystemExit(f"unknown case {a.case}")
    torch.cuda.synchronize()
    for i in range(a.iters):
        rc = fn(i)
        assert rc == 0, rc
    torch.cuda.synchronize()
    assert ops.status() == 0
    print("ok", a.case)


if __name__ == "__main__":
    main()
