"""Pins the CPU oracle to the facts the reference's own tests hold for this path.

Each test names the reference file:line whose constants or formulas it reproduces.
CPU only.
"""
import os

import numpy as np
import pytest

import oracle

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_gemm_matches_golden_from_compiled_reference():
    # vectors produced by the reference's gemm_mma_cpu (op/cpu/cpu_ops.cpp:95-114)
    z = np.load(os.path.join(GOLD, "gemm_mma_cpu.npz"))
    for i in range(5):
        C = oracle.gemm_f32(z[f"A{i}"], z[f"B{i}"])
        assert np.array_equal(C.view(np.uint32), z[f"C{i}"].view(np.uint32)), i


@pytest.mark.skipif(oracle.ref_lib() is None, reason="compiled reference not present")
def test_gemm_bit_exact_with_compiled_reference_and_threads():
    rng = np.random.default_rng(1)
    A = rng.standard_normal((37, 513), dtype=np.float32)
    B = rng.standard_normal((29, 513), dtype=np.float32)
    ref = oracle.gemm_f32(A, B, use_reference=True)
    assert np.array_equal(oracle.gemm_f32(A, B).view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(oracle.gemm_f32(A, B, threads=4).view(np.uint32), ref.view(np.uint32))


def test_operand_convention_is_a_times_b_transposed():
    # A[M,K], B[N,K] row-major, C = A * B^T (op/cpu/cpu_ops.cpp:95-113)
    A = np.arange(6, dtype=np.float32).reshape(2, 3)
    B = np.arange(12, dtype=np.float32).reshape(4, 3) - 5
    assert np.array_equal(oracle.gemm_f32(A, B), A @ B.T)


def test_fp8_all_ones_tile_is_32():
    # op/test/arch_primitives/ptx_mma_fp8.cu:48-59: E4M3 1.0 = 0x38, m16n8k32 of ones = 32, tol 0
    L = oracle.lib()
    assert L.oracle_decode_e4m3(0x38) == 1.0
    assert L.oracle_encode_e4m3(1.0) == 0x38
    word = np.array([0x38383838], np.uint32).view(np.uint8)  # four values per b32, LSB first
    assert list(oracle.decode_e4m3(word)) == [1.0] * 4
    A = oracle.decode_e4m3(np.full((16, 32), 0x38, np.uint8))
    B = oracle.decode_e4m3(np.full((8, 32), 0x38, np.uint8))
    assert np.all(oracle.gemm_f32(A, B) == 32.0)


def test_fp8_per_tensor_scale_is_applied_after_the_accumulation():
    # op/test/arch_primitives/ptx_mma_fp8.cu:16-23: the MMA sees only qA, qB; the epilogue
    # multiplies the fp32 accumulator by scale_A * scale_B
    aq, bq, sa, sb = oracle.make_fp8_case(8, 8, 64, seed=3)
    acc = oracle.gemm_f32(oracle.decode_e4m3(aq), oracle.decode_e4m3(bq))
    full = oracle.gemm_f32(oracle.decode_e4m3(aq) * np.float32(sa), oracle.decode_e4m3(bq) * np.float32(sb))
    np.testing.assert_allclose(acc * np.float32(sa * sb), full, rtol=1e-5)


def test_e2m1_table_and_sign_bit():
    # op/test/arch_primitives/ptx_mma_fp4.cu:49-53, 285-291
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    got = oracle.decode_e2m1(np.arange(16, dtype=np.uint8))
    assert list(got[:8]) == mags and list(got[8:]) == [-m for m in mags]
    assert oracle.lib().oracle_decode_e2m1(0x3) == 1.5 and oracle.lib().oracle_decode_e2m1(0x9) == -0.5
    for code in range(16):
        v = float(got[code])
        if v != 0.0:
            assert oracle.lib().oracle_encode_e2m1(v) == code


def test_ue4m3_scale_decode():
    # op/test/arch_primitives/ptx_mma_fp4.cu:55-65, 293-309
    L = oracle.lib()
    assert [L.oracle_decode_ue4m3(b) for b in (0x30, 0x38, 0x40, 0x48)] == [0.5, 1.0, 2.0, 4.0]
    assert np.isnan(L.oracle_decode_ue4m3(0x7F))
    assert L.oracle_decode_ue4m3(0x01) == 2.0 ** -9 and L.oracle_decode_ue4m3(0x07) == 7 * 2.0 ** -9
    assert L.oracle_decode_ue4m3(0x08) == 2.0 ** -6
    assert L.oracle_decode_ue4m3(0x7E) == 448.0
    # four scale bytes per b32, little-endian
    assert int(np.array([0x30, 0x38, 0x40, 0x48], np.uint8).view(np.uint32)[0]) == 0x48403830
    assert int(np.array([0x38, 0x40, 0x30, 0x48], np.uint8).view(np.uint32)[0]) == 0x48304038


def test_nvfp4_known_answer_tile():
    # op/test/arch_primitives/ptx_mma_fp4.cu:235-283, 311-324: m16n8k64, every A nibble 0x3,
    # every B nibble 0x9, C = 0.25, block scales as below -> closed form, then RN cast to fp16
    M, N, K = 16, 8, 64
    aq = oracle.pack_u4(np.full((M, K), 0x3, np.uint8))
    bq = oracle.pack_u4(np.full((N, K), 0x9, np.uint8))
    assert int(aq.view(np.uint32)[0, 0]) == 0x33333333  # 8 nibbles / b32, element i at bits [4i+3:4i]
    sfa = np.tile(np.array([0x30, 0x38, 0x40, 0x48], np.uint8), (M, 1))
    sfb = np.tile(np.array([0x38, 0x40, 0x30, 0x48], np.uint8), (N, 1))
    A = oracle.dequant_nvfp4(aq, sfa, 1.0); B = oracle.dequant_nvfp4(bq, sfb, 1.0)
    D = oracle.gemm_f32_addc(A, B, np.full((M, N), 0.25, np.float32))
    expected = 0.25 + sum(16 * (1.5 * sa) * (-0.5 * sb) for sa, sb in zip((0.5, 1, 2, 4), (1, 2, 0.5, 4)))
    assert expected == -233.75
    assert np.all(np.abs(D - expected) <= 1e-3)   # the reference's tolerance
    assert np.all(D == expected)                  # and in fact exact
    assert oracle.decode_f16(oracle.encode_f16(D))[0, 0] == np.float16(expected)


def _a_s4(r, c): return ((r * 5 + c * 3 + 2) % 15) - 7
def _b_s4(r, c): return ((r * 2 + c * 7 + 4) % 15) - 7
def _acc(r, c): return r * 13 - c * 5 - 37


def test_int4_nibble_order_and_known_answer():
    # op/test/arch_primitives/ptx_mma_integer.cu:61-74 (values), :93-108 (packing), :387-401 (answer)
    assert list(oracle.pack_s4(np.array([-1, -7], np.int8))) == [0x9F]   # -1 -> 0xF low, -7 -> 0x9 high
    vals = np.array([1, -2, 3, -4, 5, -6, 7, -8], np.int8)
    word = int(oracle.pack_s4(vals).view(np.uint32)[0])
    for i, v in enumerate(vals):
        assert (word >> (4 * i)) & 0xF == (int(v) & 0xF)
    assert np.array_equal(oracle.unpack_s4(oracle.pack_s4(vals)), vals)
    M, N, K = 16, 8, 32
    A = np.array([[_a_s4(r, k) for k in range(K)] for r in range(M)], np.int8)
    Bt = np.array([[_b_s4(k, c) for k in range(K)] for c in range(N)], np.int8)   # B[N,K] = logical B[K,N]^T
    C0 = np.array([[_acc(r, c) for c in range(N)] for r in range(M)], np.float32)
    A2 = oracle.unpack_s4(oracle.pack_s4(A)).astype(np.float32)
    B2 = oracle.unpack_s4(oracle.pack_s4(Bt)).astype(np.float32)
    D = oracle.gemm_f32_addc(A2, B2, C0)
    for r in range(M):
        for c in range(N):
            want = _acc(r, c) + sum(_a_s4(r, k) * _b_s4(k, c) for k in range(K))
            assert D[r, c] == want


def test_sparse_24_encoding_and_known_answer():
    # op/test/arch_primitives/ptx_mma_sparse.cu:53-64 (nibbles), :128-147 (values),
    # :163-184 (compressed layout), :416-434 (dense ground truth, exact comparison)
    M, N, K = 16, 8, 32
    def ra(row, grp, idx):
        return float((row + grp) % 5 + 1) if idx == 0 else -float((row * 2 + grp) % 5 + 1)
    dense = np.zeros((M, K), np.float32)
    for r in range(M):
        for g in range(K // 4):
            dense[r, 4 * g] = ra(r, g, 0); dense[r, 4 * g + 1] = ra(r, g, 1)
    dq = oracle.encode_e4m3(dense)          # small integers: exact in E4M3
    assert np.array_equal(oracle.decode_e4m3(dq), dense)
    comp, meta = oracle.sp24_compress(dq)
    assert comp.shape == (M, K // 2) and meta.shape == (M, K // 8)
    assert np.all(meta == 0x44)             # every group keeps {0,1}: nibble 0x4, packed 0x44444444
    assert int(meta.view(np.uint32)[0, 0]) == 0x44444444
    for r in range(M):
        for g in range(K // 4):
            assert oracle.decode_e4m3(comp[r, 2 * g]) == ra(r, g, 0)
            assert oracle.decode_e4m3(comp[r, 2 * g + 1]) == ra(r, g, 1)
    assert np.array_equal(oracle.sp24_expand(comp, meta), dq)
    Bt = np.array([[float((k * 3 + c * 5 + 1) % 9 - 4) for k in range(K)] for c in range(N)], np.float32)
    C0 = np.array([[(r - c) * 0.25 for c in range(N)] for r in range(M)], np.float32)
    D = oracle.gemm_f32_addc(oracle.decode_e4m3(oracle.sp24_expand(comp, meta)), Bt, C0)
    want = dense.astype(np.float64) @ Bt.T.astype(np.float64) + C0
    assert np.array_equal(D.astype(np.float64), want)


def test_sparse_24_all_six_legal_nibbles_and_rejects():
    pairs = {(0, 1): 0x4, (0, 2): 0x8, (1, 2): 0x9, (0, 3): 0xC, (1, 3): 0xD, (2, 3): 0xE}
    for (p0, p1), nib in pairs.items():
        d = np.zeros((1, 8), np.uint8); d[0, p0] = 0x38; d[0, p1] = 0xB8; d[0, 4 + p0] = 0x40; d[0, 4 + p1] = 0x30
        comp, meta = oracle.sp24_compress(d)
        assert meta[0, 0] == (nib | (nib << 4))
        assert list(comp[0]) == [0x38, 0xB8, 0x40, 0x30]
        assert np.array_equal(oracle.sp24_expand(comp, meta), d)
    with pytest.raises(ValueError):
        oracle.sp24_compress(np.full((1, 8), 0x38, np.uint8))
    # fewer than two non-zeros: still an ascending pair, still round-trips
    for pos in range(4):
        d = np.zeros((1, 8), np.uint8); d[0, pos] = 0x38
        comp, meta = oracle.sp24_compress(d)
        assert (meta[0, 0] & 0xF) in pairs.values() and (meta[0, 0] >> 4) in pairs.values()
        assert np.array_equal(oracle.sp24_expand(comp, meta), d)


def test_output_cast_is_round_to_nearest_even():
    # op/test/arch_primitives/ptx_mma_fp4.cu:277-282 (RN cast of the fp32 accumulator at the end)
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e38, 1e-40], np.float32)
    got = oracle.decode_bf16(oracle.encode_bf16(x))
    assert got[0] == 1.0 and got[1] == 1.0 and got[2] == np.float32(1.015625)
    import torch
    t = torch.from_numpy(np.random.default_rng(0).standard_normal(4096).astype(np.float32))
    want = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.encode_bf16(t.numpy()), want)


def test_tensor_parallel_sharding_and_replica_sum():
    # op/nccl/nccl_mlp_test.cu:321-352: first weight split by output features (columns of
    # [in,out]), second by input features (a slab of rows); partial outputs sum to the whole
    rng = np.random.default_rng(5)
    X = rng.standard_normal((4, 6)).astype(np.float32)
    A = rng.standard_normal((6, 8)).astype(np.float32)
    B = rng.standard_normal((8, 5)).astype(np.float32)
    full = (X @ A) @ B
    acc = np.zeros_like(full)
    for r in range(2):
        Ar = oracle.shard_cols(A, r, 2); Br = oracle.shard_rows(B, r, 2)
        assert np.array_equal(Ar, A[:, r * 4:(r + 1) * 4]) and np.array_equal(Br, B[r * 4:(r + 1) * 4])
        acc += (X @ Ar) @ Br
    np.testing.assert_allclose(acc, full, rtol=1e-5, atol=1e-5)


def test_compare_metric_floor():
    # op/nccl/nccl_mlp_test.cu:444-458
    ma, mr = oracle.compare(np.array([1.0, 0.0], np.float32), np.array([1.5, 1e-9], np.float32))
    assert ma == 0.5 and abs(mr - 0.5 / 1.5) < 1e-6 or mr >= 1e-9 / 1e-6 - 1e-6


def test_quantisers_round_trip_and_scale_rules():
    rng = np.random.default_rng(7)
    x = rng.standard_normal((5, 64), dtype=np.float32)
    q, s = oracle.quant_rows_e4m3(x)
    assert np.allclose(s, np.abs(x).max(1) / 448.0)
    inv = (np.float32(1.0) / s).astype(np.float32)
    assert np.array_equal(q, oracle.encode_e4m3((x * inv[:, None]).astype(np.float32)))   # reciprocal-multiply rule
    assert np.abs(oracle.decode_e4m3(q) * s[:, None] - x).max() <= np.abs(x).max() * 2.0 ** -4
    g = float(np.abs(x).max() / (6 * 448))
    q4, sf = oracle.quant_nvfp4(x, g)
    assert q4.shape == (5, 32) and sf.shape == (5, 4)
    back = oracle.dequant_nvfp4(q4, sf, g)
    assert np.abs(back - x).max() <= np.abs(x).max() * 0.3
    # the block maximum maps to +-6 (or the neighbouring code when the scale rounds up)
    nib = oracle.unpack_u4(q4) & 7
    assert np.all(nib.reshape(5, 4, 16).max(-1) >= 5)


def test_row_quantiser_scale_floor_keeps_tiny_rows_finite():
    x = np.zeros((3, 16), np.float32)
    x[0, 0] = 1e-37; x[1, 1] = 9.2e-41; x[2, 2] = 1e-35
    q, s = oracle.quant_rows_e4m3(x)
    assert s[0] == np.float32(2.0 ** -126) and s[1] == np.float32(2.0 ** -126) and s[2] > np.float32(2.0 ** -126)
    assert ((q & 0x7F) != 0x7F).all() and np.isfinite(oracle.decode_e4m3(q)).all()
    assert (q[:, 8:] == 0).all()                               # zeros stay zeros


def test_w4a16_dequant_rule():
    xb, wq, s = oracle.make_w4a16_case(1, 4, 256, group=128, seed=0)
    W = oracle.dequant_w4(wq, s, 128)
    ints = oracle.unpack_s4(wq).astype(np.float32)
    sc = oracle.decode_f16(s)
    assert ints.min() >= -8 and ints.max() <= 7
    assert np.array_equal(W, ints * np.repeat(sc, 128, axis=1))
    assert sc.min() >= 0.0049 and sc.max() <= 0.0201
