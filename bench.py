#!/usr/bin/env python
"""Benchmark of the quantized-GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward pass of the tensor-parallel SwiGLU MLP of the benchmark
configuration (tokens 4096, hidden 8192, intermediate 28672, E4M3 weights with per-channel
scales, bf16 activations), sharded over N ranks (gate/up column-parallel, down row-parallel,
one sum all-reduce).  Total work is fixed as N grows ("strong" scaling).  Rank 0 prints ONE JSON
line; at N=1 it also carries the per-format GEMM cases (FP8 8192^3, W4A16 decode, ...) with
their roofline fractions, and the reference's CPU GEMM path timed on the host cores.

``--impl reference`` times the reference project's own CPU implementation of the same path
(its compiled gemm_mma_cpu from oracle/_ref when present, else the C restatement in oracle/)
on a bounded sample of the same workload, all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS, HIDDEN, INTER = 4096, 8192, 28672
MLP_FLOPS = 2 * TOKENS * HIDDEN * (2 * INTER) + 2 * TOKENS * INTER * HIDDEN
NOMINAL = {"fp8_tflops": 4500.0, "fp4_tflops": 9000.0, "hbm_gbs": 7700.0}


def measured_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p)); d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock, power and throttle reasons while the timed region runs (read-only NVML
    queries every few milliseconds; nvidia-smi polling as the fallback)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.stop_flag, self.thread = index, [], None, False, None
        self.nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[self.index]) if vis and vis.split(",")[self.index].isdigit() else self.index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.nvml = pynvml
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._poll, daemon=True); self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True); self.thread.start()
        except Exception:
            self.proc = None

    def _poll(self):
        n = self.nvml
        names = {"hw_slowdown": n.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": n.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": n.nvmlClocksThrottleReasonSwThermalSlowdown,
                 "sw_power_cap": n.nvmlClocksThrottleReasonSwPowerCap}
        while not self.stop_flag:
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                pw = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                rs = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.rows.append((float(sm), float(self.max_sm), pw, [k for k, bit in names.items() if rs & bit]))
            except Exception:
                pass
            time.sleep(0.004)

    def _read(self):
        for line in self.proc.stdout:
            r = [c.strip() for c in line.split(",")]
            try:
                reasons = [nm for nm, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9])
                           if v.lower().startswith("active")]
                self.rows.append((float(r[1]), float(r[2]), float(r[3]), reasons))
            except Exception:
                continue

    def stop(self) -> dict:
        self.stop_flag = True
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        if self.thread is not None:
            self.thread.join(timeout=2)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        pw = [r[2] for r in self.rows]
        busy = [r for r in self.rows if r[2] >= 0.6 * max(pw)] or self.rows      # samples taken under load
        reasons = sorted({x for r in busy for x in r[3]})
        return {"sm_mhz": statistics.median(r[0] for r in busy), "sm_max_mhz": max(r[1] for r in self.rows),
                "power_w_max": max(pw), "samples": len(self.rows), "samples_under_load": len(busy),
                "reasons": reasons, "source": "nvml" if self.nvml else "nvidia-smi"}


# ------------------------------------------------------------------ CPU reference arm

def cpu_mlp_sample(n_tokens: int, weights_host, x_host, threads: int, use_ref: bool):
    """The whole MLP for ``n_tokens`` tokens on the host, every GEMM by the reference's CPU loop."""
    import numpy as np
    import oracle
    wg, sg, wu, su, wd, sd = weights_host
    x = oracle.decode_bf16(x_host[:n_tokens])
    t0 = time.perf_counter()
    xq, sx = oracle.quant_rows_e4m3(x)
    X = oracle.decode_e4m3(xq)
    g = oracle.gemm_f32(X, wg, threads=threads, use_reference=use_ref) * (sx[:, None] * sg[None, :])
    u = oracle.gemm_f32(X, wu, threads=threads, use_reference=use_ref) * (sx[:, None] * su[None, :])
    h = oracle.decode_bf16(oracle.encode_bf16(oracle.swiglu(g, u)))
    hq, sh = oracle.quant_rows_e4m3(h)
    y = oracle.gemm_f32(oracle.decode_e4m3(hq), wd, threads=threads, use_reference=use_ref) * (sh[:, None] * sd[None, :])
    dt = time.perf_counter() - t0
    return dt, oracle.encode_bf16(y)


def cpu_single_thread(weights, x_host_u16, use_ref: bool, n_tokens: int) -> dict:
    """gemm_mma_cpu as the reference ships it: one thread (op/cpu/cpu_ops.cpp:95-114 has no threading)."""
    dt, _ = cpu_mlp_sample(n_tokens, weights, x_host_u16, 1, use_ref)
    return {"value": n_tokens / dt, "unit": "tokens/s", "cores": 1,
            "sample": f"{n_tokens} of {TOKENS} tokens through the whole MLP, {dt:.1f} s, "
                      f"{MLP_FLOPS / TOKENS * n_tokens / dt / 1e9:.2f} GFLOP/s"}


def host_weights(seed: int = 0):
    """E4M3 weights N(0,1) with per-output-channel scales U(0.001, 0.01), decoded to fp32 for the CPU arm."""
    import numpy as np
    import oracle
    rng = np.random.default_rng(seed)

    def w(rows, cols):
        q = oracle.encode_e4m3(rng.standard_normal((rows, cols), dtype=np.float32))
        return oracle.decode_e4m3(q), rng.uniform(0.001, 0.01, rows).astype(np.float32)
    wg, sg = w(INTER, HIDDEN); wu, su = w(INTER, HIDDEN); wd, sd = w(HIDDEN, INTER)
    return wg, sg, wu, su, wd, sd


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import oracle
    oracle.build()
    use_ref = oracle.ref_lib() is not None
    cores = os.cpu_count() or 1
    weights = host_weights()
    rng = np.random.default_rng(1)
    sample = args.cpu_tokens
    x = oracle.encode_bf16(rng.standard_normal((sample, HIDDEN), dtype=np.float32))
    times = []
    for i in range(args.warmup + args.steps):
        dt, _ = cpu_mlp_sample(sample, weights, x, cores, use_ref)
        if i >= args.warmup:
            times.append(dt)
    t = sum(times) / len(times)
    val = sample / t
    desc = {"value": val, "unit": "tokens/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"{sample} of {TOKENS} tokens through the whole MLP per step (all GEMMs by gemm_mma_cpu on "
                      f"row blocks, one thread per core); GFLOP/s = {MLP_FLOPS / TOKENS * sample / t / 1e9:.2f}",
            "single_thread": cpu_single_thread(weights, x, use_ref, args.cpu_tokens_single)}
    print(json.dumps({
        "impl": "reference", "metric": "tp_mlp_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": desc,
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(n):
    """The `config` object of the JSON line: the same keys and values in both arms."""
    return {"workload": f"SwiGLU TP-MLP tokens={TOKENS} hidden={HIDDEN} intermediate={INTER}, E4M3 weights + "
                        f"per-channel fp32 scales, bf16 activations, tp{n}",
            "tokens": TOKENS, "hidden": HIDDEN, "intermediate": INTER, "parallelism": f"tp{n}",
            "l2": "per-rank weights + activations exceed the 126 MB L2 every step"}


def recorded_profile(kernel_key: str):
    """Figures that only a profiler can give (DRAM traffic, tensor-pipe activity) are not measured by this
    program: they are read from profiles/recorded_counters.json, which names the ncu summary and the commit
    each one was taken at.  Missing file or key -> None."""
    try:
        with open(os.path.join(ROOT, "profiles", "recorded_counters.json")) as f:
            return json.load(f).get(kernel_key)
    except Exception:
        return None


# ------------------------------------------------------------------------- GPU arm

def time_graph(fn, iters: int, reps: int = 5):
    """Captures ``iters`` calls of fn() into one CUDA graph and returns the best ms per call."""
    import torch
    fn(); torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i)
    g.replay(); torch.cuda.synchronize()
    best = 1e30
    for _ in range(reps):
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(); g.replay(); e1.record(); torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / iters)
    return best


def time_loop(fn, iters: int, warm: int = 3):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _e4m3_normal(rows, cols, gen):
    """N(0,1) scaled to fit +-448 with one per-tensor scale, as E4M3 bytes (the FP8 GEMM configuration)."""
    import torch
    x = torch.randn((rows, cols), device="cuda", generator=gen)
    scale = float(x.abs().max()) / 448.0
    return (x / scale).to(torch.float8_e4m3fn).view(torch.uint8), scale


def _nvfp4_normal(rows, K, gen):
    """N(0,1) quantised to NVFP4: E2M1 codes packed two per byte (low nibble = lower K), one UE4M3 scale per
    16 K (block max-abs / 6, relative to one fp32 global scale), as the NVFP4 configuration states."""
    import torch
    x = torch.randn((rows, K // 16, 16), device="cuda", generator=gen)
    amax = x.abs().amax(-1)
    glob = float(amax.max()) / (6.0 * 448.0)
    sf = (amax / 6.0 / glob).to(torch.float8_e4m3fn)
    y = x / (sf.float() * glob).clamp_min(1e-30).unsqueeze(-1)
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device="cuda")
    code = torch.bucketize(y.abs(), mids).to(torch.uint8) | ((y < 0).to(torch.uint8) << 3)
    code = code.view(rows, K)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), sf.view(torch.uint8).contiguous(), glob


def _sparse24_normal(rows, K, gen):
    """2:4 sparse A: in every 4 consecutive K two positions chosen uniformly, values N(0,1) as E4M3 with a
    per-tensor scale; returns the compressed values [rows, K/2], the metadata bytes [rows, K/8] and the scale."""
    import torch
    vals, scale = _e4m3_normal(rows, K // 2, gen)
    pairs = torch.tensor([0b0100, 0b1000, 0b1100, 0b1001, 0b1101, 0b1110], dtype=torch.uint8, device="cuda")  # (p0 | p1 << 2), p0 < p1
    pick = torch.randint(0, 6, (rows, K // 4), device="cuda", generator=gen)
    nib = pairs[pick]
    meta = nib[:, 0::2] | (nib[:, 1::2] << 4)
    return vals, meta.contiguous(), scale


def gemm_cases(peaks):
    """Per-format GEMM numbers (rank 0, N=1): TFLOPS or GB/s and fractions of nominal / measured peaks."""
    import torch
    import cudaop_b200 as ops
    L = ops.lib()
    import time
    out = {"note": "each case is a kernel timed alone after the GPU idled for a second or more (burst clocks, the regime of "
                   "the bf16_tflops / hbm_gbs peaks it is compared with); the MLP step above runs in the sustained regime"}
    st = lambda: torch.cuda.current_stream().cuda_stream
    fp8_meas = 2.0 * peaks["bf16_tflops"]
    torch.cuda.synchronize(); time.sleep(3.0)
    # FP8 8192^3 (operands 128 MB > L2 is not true here: 2 x 64 MB + 128 MB C; C alone exceeds L2)
    S = 8192
    gen = torch.Generator(device="cuda").manual_seed(0)
    a, sa = _e4m3_normal(S, S, gen)
    b, sb = _e4m3_normal(S, S, gen)
    c = torch.empty((S, S), dtype=torch.bfloat16, device="cuda")
    ms = time_loop(lambda: L.b200q_gemm_fp8(a.data_ptr(), b.data_ptr(), c.data_ptr(), S, S, S, sa, sb, st()), 20)
    tf = 2 * S ** 3 / ms / 1e9
    out["fp8_8192"] = {"ms": ms, "tflops": tf, "frac_nominal_4500": tf / NOMINAL["fp8_tflops"],
                       "frac_2x_measured_bf16": tf / fp8_meas}
    # the same kernel on operands of lower switching activity (uniform bytes in [0,120): positive, all exponents):
    # the part runs at its power cap, so the operand statistics set the clock and with it the TFLOPS
    torch.cuda.synchronize(); time.sleep(1.5)
    a.copy_(torch.randint(0, 120, (S, S), dtype=torch.uint8, device="cuda", generator=gen))
    b.copy_(torch.randint(0, 120, (S, S), dtype=torch.uint8, device="cuda", generator=gen))
    torch.cuda.synchronize(); time.sleep(1.0)
    ms = time_loop(lambda: L.b200q_gemm_fp8(a.data_ptr(), b.data_ptr(), c.data_ptr(), S, S, S, 1.0, 1.0, st()), 20)
    tf = 2 * S ** 3 / ms / 1e9
    out["fp8_8192_uniform_bytes"] = {"ms": ms, "tflops": tf, "frac_nominal_4500": tf / NOMINAL["fp8_tflops"],
                                     "frac_2x_measured_bf16": tf / fp8_meas,
                                     "note": "not the configuration's distribution: shows the power-cap effect of the data"}
    del a, b, c
    torch.cuda.synchronize(); time.sleep(1.5)
    # NVFP4 8192^3 (scales pre-blocked, as weights would be)
    A4, sfa_rm, ga = _nvfp4_normal(S, S, gen)
    B4, sfb_rm, gb = _nvfp4_normal(S, S, gen)
    sfa = ops.nvfp4_swizzle_sf(sfa_rm, S); sfb = ops.nvfp4_swizzle_sf(sfb_rm, S)
    c = torch.empty((S, S), dtype=torch.bfloat16, device="cuda")
    ms = time_loop(lambda: L.b200q_gemm_nvfp4_blocked(A4.data_ptr(), sfa.data_ptr(), B4.data_ptr(), sfb.data_ptr(), c.data_ptr(),
                                                      S, S, S, ga, gb, st()), 20)
    tf = 2 * S ** 3 / ms / 1e9
    out["nvfp4_8192"] = {"ms": ms, "tflops": tf, "frac_nominal_9000": tf / NOMINAL["fp4_tflops"],
                         "frac_4x_measured_bf16": tf / (4.0 * peaks["bf16_tflops"])}
    del A4, B4, sfa, sfb, sfa_rm, sfb_rm
    torch.cuda.synchronize(); time.sleep(1.5)
    # MXFP8 8192^3 (E4M3 data, one UE8M0 scale per 32 K; scales pre-blocked)
    xa = torch.randn((S, S // 32, 32), device="cuda", generator=gen); xb = torch.randn((S, S // 32, 32), device="cuda", generator=gen)

    def mx(x):
        e = torch.floor(torch.log2(x.abs().amax(-1).clamp_min(2.0 ** -100))) - 8.0
        q = (x * torch.exp2(-e).unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        return q.view(S, S).contiguous(), (e + 127.0).to(torch.uint8).contiguous()
    A8, sa8 = mx(xa); B8, sb8 = mx(xb)
    del xa, xb
    sa8b = ops.mxfp8_swizzle_sf(sa8, S); sb8b = ops.mxfp8_swizzle_sf(sb8, S)
    ms = time_loop(lambda: L.b200q_gemm_mxfp8_blocked(A8.data_ptr(), sa8b.data_ptr(), B8.data_ptr(), sb8b.data_ptr(), c.data_ptr(),
                                                      S, S, S, st()), 20)
    tf = 2 * S ** 3 / ms / 1e9
    out["mxfp8_8192"] = {"ms": ms, "tflops": tf, "frac_nominal_4500": tf / NOMINAL["fp8_tflops"], "frac_2x_measured_bf16": tf / fp8_meas}
    del A8, B8, sa8, sb8, sa8b, sb8b
    torch.cuda.synchronize(); time.sleep(1.5)
    # 2:4 sparse FP8 4096 x 8192 x 8192 (dense-equivalent FLOPs)
    Ms = 4096
    Ac, Em, ssa = _sparse24_normal(Ms, S, gen)
    Bd, ssb = _e4m3_normal(S, S, gen)
    ms = time_loop(lambda: L.b200q_gemm_sp24_fp8(Ac.data_ptr(), Em.data_ptr(), Bd.data_ptr(), c.data_ptr(), Ms, S, S, ssa, ssb, st()), 20)
    tf = 2 * Ms * S * S / ms / 1e9
    out["sparse_fp8_4096x8192x8192"] = {"ms": ms, "tflops_dense_equivalent": tf, "frac_nominal_dense_4500": tf / NOMINAL["fp8_tflops"],
                                        "frac_nominal_sparse_9000": tf / (2 * NOMINAL["fp8_tflops"])}
    del Ac, Em, Bd, c
    torch.cuda.synchronize(); time.sleep(1.5)
    # W4A16 decode: 80 distinct weight sets (671 MB > L2) cycled inside one CUDA graph
    N = K = 4096
    nsets = 80
    wq = torch.randint(0, 256, (nsets, N, K // 2), dtype=torch.uint8, device="cuda")
    sc = (torch.rand((nsets, N, K // 128), device="cuda") * 0.015 + 0.005).to(torch.float16)
    for M in (1, 16):
        x = torch.randn((M, K), device="cuda").to(torch.bfloat16)
        y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")

        def call(i=0):
            j = i % nsets
            L.b200q_gemm_w4a16(x.data_ptr(), wq[j].data_ptr(), sc[j].data_ptr(), y.data_ptr(), M, N, K, 128, st())
        byts = N * K // 2 + N * (K // 128) * 2 + 2 * M * K + 2 * M * N
        ms = time_graph(call, 2 * nsets)
        gbs = byts / ms / 1e6
        out[f"w4a16_m{M}"] = {"us": ms * 1e3, "gbs": gbs, "frac_measured_hbm": gbs / peaks["hbm_gbs"],
                              "frac_nominal_7700": gbs / NOMINAL["hbm_gbs"], "bytes": byts,
                              "note": "80 distinct weight sets cycled in one CUDA graph"}
        if M == 1:
            # the same with programmatic dependent launch: a call streams its weights while the one before it drains
            L.b200q_w4a16_set_pdl(1)
            ms = time_graph(call, 2 * nsets)
            L.b200q_w4a16_set_pdl(0)
            gbs = byts / ms / 1e6
            out["w4a16_m1_pdl"] = {"us": ms * 1e3, "gbs": gbs, "frac_measured_hbm": gbs / peaks["hbm_gbs"],
                                   "frac_nominal_7700": gbs / NOMINAL["hbm_gbs"], "bytes": byts,
                                   "note": "as w4a16_m1, calls chained with programmatic dependent launch (b200q_w4a16_set_pdl)"}
    # W4A16 at a prefill shape: 4096 tokens (tcgen05 kernel, integer weights, group scales on the fp32 partial sums)
    Mp = 4096
    xp = torch.randn((Mp, K), device="cuda").to(torch.bfloat16)
    yp = torch.empty((Mp, N), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize(); time.sleep(1.0)
    ms = time_loop(lambda: L.b200q_gemm_w4a16(xp.data_ptr(), wq[0].data_ptr(), sc[0].data_ptr(), yp.data_ptr(), Mp, N, K, 128, st()), 20)
    tf = 2 * Mp * N * K / ms / 1e9
    out["w4a16_prefill_4096"] = {"ms": ms, "tflops": tf, "frac_nominal_bf16_2250": tf / 2250.0, "frac_measured_bf16": tf / peaks["bf16_tflops"]}
    del wq, sc, xp, yp
    torch.cuda.empty_cache()
    return out


def multi_rank_parity(mlp, x, rank, world, dev):
    """Outside the timed loops: one forward in the timed mode, checked the way the reference checks the run it
    times (op/nccl/nccl_mlp_test.cu:625-664: replicas equal, result against an independent computation).
    * replicas_equal: every rank's Y is bit-identical to rank 0's;
    * exact_frac / max_ulp_vs_rank_order_sum: Y against the fp32 sum, in rank order, of the gathered partials,
      rounded once to bf16 (peer loads must match bit for bit; the in-switch reduction may differ by one ulp);
    * h_rows_rel_fro: 64 sampled rows of this run's H (rank 0's shard) against a float64 product of the same
      quantised operands on the host."""
    import torch
    import torch.distributed as dist
    y = mlp.forward(x); mlp.wait()
    torch.cuda.synchronize()
    y = y.clone()
    if mlp.comm == "nccl":          # NCCL reduced the partial in place: rebuild this rank's own with the stand-alone GEMM
        import cudaop_b200 as ops
        mine = ops.gemm_fp8_rowcol(mlp.hq[:TOKENS], mlp.wd, mlp.shs[:TOKENS], mlp.sd, out_dtype=torch.float32)
    else:
        mine = mlp.partial[:TOKENS].contiguous()
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    acc = torch.zeros((TOKENS, HIDDEN), dtype=torch.float32, device=dev)
    for p_ in parts:
        acc += p_.float()
    del parts
    want = acc.to(torch.bfloat16)
    y0 = y.clone()
    dist.broadcast(y0, src=0)
    eq = torch.tensor([int(torch.equal(y, y0))], device=dev)
    dist.all_reduce(eq, op=dist.ReduceOp.MIN)
    wf, yf = want.float(), y.float()
    ulp = torch.maximum(wf.abs(), torch.full_like(wf, 2.0 ** -120)).log2().floor().exp2() * 2.0 ** -7
    # in bf16 ulps of the rank-order sum itself; sums that cancelled to (almost) nothing are left out of the ratio
    big = wf.abs() >= 2.0 ** -20 * wf.abs().max()
    dist_ulp = ((yf - wf).abs() / ulp)[big].max()
    out = {"replicas_equal": bool(eq.item()), "exact_frac": float((y == want).float().mean().item()),
           "max_ulp_vs_rank_order_sum": float(dist_ulp.item()),
           "transport": ("copy engines both ways, local sum kernel" if mlp.comm == "pipelined_copy" else
                         ("multimem (in-switch reduction)" if getattr(mlp, "multicast", False) else "peer loads/stores") +
                         (", result gathered by copy engines" if mlp.comm == "pipelined_ce" else "")),
           "comm": mlp.comm}
    if rank == 0:
        g = torch.Generator().manual_seed(11)
        rows = torch.randperm(TOKENS, generator=g)[:64].to(dev)
        e4 = lambda t: t.view(torch.float8_e4m3fn).to(torch.float64).cpu()
        xq, sx = e4(mlp.xq[rows]), mlp.sx[rows].double().cpu()
        gg = (xq @ e4(mlp.wg).T) * (sx[:, None] * mlp.sg.double().cpu()[None, :])
        uu = (xq @ e4(mlp.wu).T) * (sx[:, None] * mlp.su.double().cpu()[None, :])
        ref = (gg / (1.0 + torch.exp(-gg)) * uu)
        got = mlp.h[rows].double().cpu()
        ref_b = ref.to(torch.bfloat16).double()             # the same final cast as the kernel's
        out["h_rows_rel_fro"] = float(((got - ref_b).norm() / ref_b.norm()).item())
        out["h_rows_rel_fro_raw"] = float(((got - ref).norm() / ref.norm()).item())
    return out


def run_ours(args):
    # everything that libraries print (NCCL's version banner, warnings) goes to stderr: stdout
    # carries the one JSON line only
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    import torch
    import torch.distributed as dist
    import cudaop_b200 as ops
    from cudaop_b200.mlp import TensorParallelMLP

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)
    ops.lib()   # fails loudly if the CUDA library is missing
    if args.static_tiles:
        ops.lib().b200q_fp8_set_dynamic_tiles(0)
    peaks = measured_peaks()

    # synthetic weights, generated shard by shard on the device from per-row seeds so that every
    # world size multiplies the same matrices
    loc = INTER // world
    gen = torch.Generator(device=dev)

    def rand_e4m3(rows, cols, seed):
        gen.manual_seed(seed)
        return torch.randn((rows, cols), device=dev, generator=gen).to(torch.float8_e4m3fn).view(torch.uint8)

    def rand_scale(n, seed):
        gen.manual_seed(seed)
        return torch.rand((n,), device=dev, generator=gen) * 0.009 + 0.001
    # shard r of gate/up = block r of `world` equal row blocks; generate only this rank's block
    wg = rand_e4m3(loc, HIDDEN, 1000 + rank) ; wu = rand_e4m3(loc, HIDDEN, 2000 + rank)
    wd = rand_e4m3(HIDDEN, loc, 3000 + rank)
    sg = rand_scale(loc, 4000 + rank); su = rand_scale(loc, 5000 + rank); sd = rand_scale(HIDDEN, 6000)
    mlp = TensorParallelMLP(wg, sg, wu, su, wd, sd, rank=rank, world=world, device=dev, max_tokens=TOKENS,
                            chunks=args.chunks if world > 1 else 1, presharded=True, comm=args.comm,
                            ar_ctas=args.ar_ctas, use_multicast={"auto": None, "on": True, "off": False}[args.multicast],
                            partial_dtype=torch.float32 if args.partial == "fp32" else torch.bfloat16)
    del wg, wu, wd

    gen.manual_seed(7)
    x_host = torch.randn((TOKENS, HIDDEN), generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).pin_memory()
    y_host = torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16).pin_memory()
    x = x_host.to(dev, non_blocking=True)
    y = torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16, device=dev)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, warmup, finish=None):
        for _ in range(warmup):
            fn()
        if finish:
            finish()
        sync_all()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if finish:
            finish()            # the timed stream waits for every side-stream all-reduce of the K steps
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    # ---- device-resident steps (the headline `value`) with events around the top kernel
    mlp.top_kernel_events = []
    def device_step():
        mlp.forward(x)
        if not args.no_prepare:       # the next (independent) batch is quantised beside this batch's GEMMs
            mlp.prepare(x)
    ms_step = timed(device_step, args.steps, args.warmup, finish=mlp.wait)
    mlp.cancel_prepared()
    evs = mlp.top_kernel_events; mlp.top_kernel_events = None
    torch.cuda.synchronize()
    top_ms = [a.elapsed_time(b) for a, b in evs[-args.steps * max(1, mlp.chunks if world > 1 else 1):]]
    launches = mlp.kernel_launches_per_forward * args.steps
    # ---- one more pass with events around every kernel (not part of the timed region)
    mlp.stage_events = []
    for _ in range(3):
        mlp.forward(x)
    torch.cuda.synchronize()
    names = ("quant_x", "gate_up_swiglu", "quant_h", "down_allreduce" if world > 1 else "down")
    kernels_ms = {n: min(m[i].elapsed_time(m[i + 1]) for m in mlp.stage_events) for i, n in enumerate(names)}
    mlp.stage_events = None
    # ---- latency of ONE forward with nothing else in flight (N > 1: the fused GEMM + all-reduce kernel)
    if world > 1:
        lat = TensorParallelMLP(mlp.wg, mlp.sg, mlp.wu, mlp.su, mlp.wd, mlp.sd, rank=rank, world=world, device=dev,
                                max_tokens=TOKENS, presharded=True, comm="fused", use_multicast=mlp.use_multicast,
                                partial_dtype=mlp.partial_dtype)
        ms_latency = timed(lambda: lat.forward(x), args.steps, args.warmup)
    else:
        ms_latency = ms_step
    # ---- end to end through the package's host-fed pipeline (cudaop_b200.mlp.HostFedMLP): every step takes its
    # input from pinned host memory and leaves its result there.  With R ranks each rank moves 1/R of X over its own
    # PCIe link, the ranks complete each other's X over NVLink (copy engines, ordered by a stream barrier), and each
    # rank writes back 1/R of the replicated result.  Copies are double-buffered on their own streams.
    from cudaop_b200.mlp import HostFedMLP
    fed = HostFedMLP(mlp, TOKENS, prepare_ahead=not args.no_prepare)

    def e2e_step():
        fed.step(x_host, y_host)
    e2e_finish = fed.finish
    ms_e2e = timed(e2e_step, args.steps, args.warmup, finish=e2e_finish)
    clocks = sampler.stop() if sampler else None
    assert ops.status() == 0, "a kernel gave up on a bounded wait"
    # what the host-fed steps left in pinned memory (this rank's rows) against a plain device-resident forward
    mlp.cancel_prepared()
    y_dev = mlp.forward(x); mlp.wait(); torch.cuda.synchronize()
    e2e_rows_equal = bool(torch.equal(y_host[fed.lo:fed.hi], y_dev[fed.lo:fed.hi].cpu()))
    parity = multi_rank_parity(mlp, x, rank, world, dev) if world > 1 else None
    if parity is not None:
        # the bar: identical replicas; peer loads / copy engines bit for bit the rank-order sum, the in-switch
        # reduction within one bf16 ulp of it.  A run that misses it still prints its line, then exits non-zero.
        exact_needed = "multimem" not in parity["transport"] and mlp.comm != "nccl"
        parity["ok"] = bool(parity["replicas_equal"] and parity["max_ulp_vs_rank_order_sum"] <= 1.0 and
                            (parity["exact_frac"] == 1.0 or not exact_needed))

    if rank != 0:
        if world > 1:
            dist.barrier(); dist.destroy_process_group()
        return

    top_avg = sum(top_ms) / max(1, len(top_ms))
    chunks = mlp.chunks if world > 1 else 1
    top_flops = 2 * (TOKENS // chunks) * HIDDEN * (2 * loc)
    top_tf = top_flops / top_avg / 1e9 if top_avg > 0 else 0.0
    peak_burst = 2.0 * peaks["bf16_tflops"]
    peak_sustained = 2.0 * peaks["bf16_tflops_sustained"]
    rec = recorded_profile("gemm_fp8_2cta_kernel_swiglu_tp1") if world == 1 else None
    line = {
        "metric": "tp_mlp_tokens_per_s", "value": TOKENS / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> fp32 acc -> bf16",
        "data": "synthetic", "config": workload_config(world),
        "tile_scheduling": "static" if args.static_tiles else "dynamic",
        "transport": {"comm": mlp.comm, "multicast": getattr(mlp, "multicast", None), "chunks": mlp.chunks,
                      "partial_dtype": str(mlp.partial_dtype).replace("torch.", "")},
        "parity": parity,
        "tflops": MLP_FLOPS / (ms_step * 1e-3) / 1e12,
        "clocks": clocks,
        "e2e": {"value": TOKENS / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": TOKENS * HIDDEN * 2, "d2h_bytes_per_step": TOKENS * HIDDEN * 2,
                "result_rows_equal_device_run": e2e_rows_equal,
                "note": "whole-job bytes per step through cudaop_b200.mlp.HostFedMLP; copies run on their own streams, "
                        "double-buffered, overlapping the GEMMs of the neighbouring steps; with R ranks each rank copies "
                        "1/R of X in and 1/R of Y out over its own PCIe link and pulls the rest of X from its peers "
                        "over NVLink (copy engines) behind a stream-ordered rank barrier"},
        "latency_ms_per_forward": ms_latency,
        "overlap": (("steps are independent batches: the all-reduce of step i runs on a side stream under the GEMMs "
                     "of step i+1 (double-buffered); latency_ms_per_forward is one forward alone with the all-reduce "
                     "fused into the down-projection kernel; ") if world > 1 and mlp.comm.startswith("pipelined") else "") +
                   ("the activation quantiser of batch i+1 runs on a side stream beside the GEMMs of batch i "
                    "(TensorParallelMLP.prepare); every step still launches it once" if not args.no_prepare else
                    "none between batches"),
        "gpu_launches": launches, "kernels_ms": kernels_ms,
        "roofline": {"bound": "tensor", "kernel": "gemm_fp8_2cta_kernel<SwiGLU> (gate/up projection, CTA pairs)",
                     "achieved": top_tf, "peak": peak_burst, "unit": "TFLOP/s", "frac": top_tf / peak_burst,
                     "peak_source": f"2 x bf16_tflops (burst) of {peaks['source']}: FP8 runs at twice the bf16 rate on "
                                    "the same tensor pipe and the driver measures no FP8 figure; the timed region is "
                                    f"{ms_step * args.steps:.0f} ms, far shorter than the seconds-long loop behind the "
                                    "sustained figure",
                     "frac_vs_2x_burst": top_tf / peak_burst, "frac_vs_2x_sustained": top_tf / peak_sustained,
                     "timed_region_ms": ms_step * args.steps,
                     "frac_nominal_4500": top_tf / NOMINAL["fp8_tflops"], "launch_ms": top_avg,
                     "flops_per_launch": top_flops,
                     "tflop_per_s_at_sampled_mhz": {"sm_mhz": clocks.get("sm_mhz") if clocks else None,
                                                    "flop_per_sm_clock": (top_flops / (top_avg * 1e-3) / (clocks["sm_mhz"] * 1e6) / 148.0)
                                                    if clocks and clocks.get("sm_mhz") else None,
                                                    "note": "8192 dense FP8 FLOP per SM and clock is the tensor pipe's rate"},
                     # profiler-only figures: recorded, not measured here (see recorded_profile)
                     "traffic": rec["dram_bytes"] if rec else None,
                     "traffic_source": rec if rec else None},
    }
    if world == 1 and not args.no_cases:
        line["cases"] = gemm_cases(peaks)
    if world == 1 and not args.no_cpu:
        import oracle
        oracle.build()
        use_ref = oracle.ref_lib() is not None
        cores = os.cpu_count() or 1
        weights = host_weights()
        import numpy as np
        xs = x_host[:args.cpu_tokens].view(torch.int16).numpy().view(np.uint16)
        dt, _ = cpu_mlp_sample(args.cpu_tokens, weights, xs, cores, use_ref)
        line["cpu_baseline"] = {"value": args.cpu_tokens / dt, "unit": "tokens/s", "cores": cores,
                                "kind": "reference" if use_ref else "port",
                                "sample": f"{args.cpu_tokens} of {TOKENS} tokens through the whole MLP, "
                                          f"{dt:.1f} s, {MLP_FLOPS / TOKENS * args.cpu_tokens / dt / 1e9:.2f} GFLOP/s",
                                "single_thread": cpu_single_thread(weights, xs, use_ref, args.cpu_tokens_single)}
    os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier(); dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        print(f"multi-rank parity check failed: {parity}", file=sys.stderr)
        sys.exit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--chunks", type=int, default=4, help="token chunks for all-reduce overlap (N > 1)")
    ap.add_argument("--comm", default="pipelined", choices=["auto", "pipelined", "pipelined_ce", "pipelined_copy", "fused", "symm", "nccl"],
                    help="all-reduce: the library's NVSwitch kernel over symmetric memory, or NCCL")
    ap.add_argument("--ar-ctas", type=int, default=None, help="CTAs of the stand-alone all-reduce kernel (default: by transport)")
    ap.add_argument("--partial", default="bf16", choices=["bf16", "fp32"], help="dtype of the partial outputs that cross NVLink")
    ap.add_argument("--multicast", default="auto", choices=["auto", "on", "off"],
                    help="reduce and broadcast in the NVSwitch (multimem) instead of peer loads/stores; auto = from 4 ranks on")
    ap.add_argument("--cpu-tokens", type=int, default=64, help="tokens in the CPU-baseline sample")
    ap.add_argument("--cpu-tokens-single", type=int, default=4, help="tokens in the single-thread CPU sample")
    ap.add_argument("--no-prepare", action="store_true",
                    help="quantise each batch inside its own forward instead of beside the previous batch's GEMMs")
    ap.add_argument("--static-tiles", action="store_true",
                    help="CTA-pair FP8 kernels with fixed round-robin tile shares instead of the global tile counter")
    ap.add_argument("--no-cases", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
