"""The cross-rank flag protocol, the reducers and the give-up path of the bounded waits on ONE GPU.

Every "rank" of a small world runs inside one cooperative launch on buffers of the same device
(b200q_*_one_device), so the code the multi-GPU runs use is exercised where only one GPU is visible.
Contract checked: fp32 sum of the partials in rank order, one round-to-nearest-even to bf16, identical
replicas (the reference asserts the same of its all-reduce, op/nccl/nccl_mlp_test.cu:181-195,646-664).
Nothing here faults or hangs a GPU: the one test that lets a wait run out does so on a flag nobody
raises, with a 5 ms limit, and reads the status word the kernel leaves.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from tests.util import dev

pytestmark = pytest.mark.gpu


def _ptr_table(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


def _host_table(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _rank_order_sum(parts):
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        acc += p.float()
    return acc.to(torch.bfloat16)


@pytest.mark.parametrize("pdt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [2, 4])
def test_allreduce_kernel_all_ranks_in_one_launch(world, pdt):
    import cudaop_b200 as ops
    L = ops.lib()
    g = torch.Generator(device="cuda").manual_seed(100 + world)
    elems = 8 * world * 1531                                  # not a multiple of the CTA's stride
    parts = [torch.randn(elems, device="cuda", generator=g).to(pdt) for _ in range(world)]
    outs = [torch.full((elems,), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(L.b200q_allreduce_signal_bytes() // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    tp, to, tf = _ptr_table(parts), _ptr_table(outs), _ptr_table(flags)
    st = torch.cuda.current_stream().cuda_stream
    want = _rank_order_sum(parts)
    for epoch in (1, 2, 3):                                   # flags are reused with a growing epoch
        for o in outs:
            o.fill_(float("nan"))
        rc = L.b200q_allreduce_to_bf16_one_device(tp.data_ptr(), to.data_ptr(), tf.data_ptr(), int(pdt == torch.bfloat16),
                                                  0, elems, world, epoch, 0, 3, st)
        assert rc == 0
        torch.cuda.synchronize()
        assert ops.status() == 0
        for o in outs:
            assert torch.equal(o, want)                       # bit exact, every replica


@pytest.mark.parametrize("pdt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [2, 4])
def test_reduce_scatter_kernel_all_ranks_in_one_launch(world, pdt):
    """The reduce-scatter half: rank r's output holds its 1/world of the sum and nothing else is touched."""
    import cudaop_b200 as ops
    L = ops.lib()
    g = torch.Generator(device="cuda").manual_seed(200 + world)
    elems = 8 * world * 1531
    per = elems // world
    parts = [torch.randn(elems, device="cuda", generator=g).to(pdt) for _ in range(world)]
    outs = [torch.full((elems,), -7.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(L.b200q_allreduce_signal_bytes() // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    tp, to, tf = _ptr_table(parts), _ptr_table(outs), _ptr_table(flags)
    st = torch.cuda.current_stream().cuda_stream
    want = _rank_order_sum(parts)
    for epoch in (1, 2):
        rc = L.b200q_reduce_scatter_to_bf16_one_device(tp.data_ptr(), to.data_ptr(), tf.data_ptr(), int(pdt == torch.bfloat16),
                                                       0, elems, world, epoch, 0, 3, st)
        assert rc == 0
        torch.cuda.synchronize()
        assert ops.status() == 0
        for r, o in enumerate(outs):
            assert torch.equal(o[r * per:(r + 1) * per], want[r * per:(r + 1) * per])
            rest = torch.cat([o[:r * per], o[(r + 1) * per:]])
            assert bool((rest == -7.0).all())


@pytest.mark.parametrize("pdt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [1, 2, 8])
def test_local_sum_kernel(n, pdt):
    """b200q_sum_to_bf16: fp32 sum in index order of n local arrays, one rounding (the arithmetic of the exchange
    when copy engines move the data)."""
    import cudaop_b200 as ops
    L = ops.lib()
    g = torch.Generator(device="cuda").manual_seed(300 + n)
    elems = 8 * 12347
    parts = [torch.randn(elems, device="cuda", generator=g).to(pdt) for _ in range(n)]
    out = torch.zeros(elems, dtype=torch.bfloat16, device="cuda")
    tp = _ptr_table(parts)
    rc = L.b200q_sum_to_bf16(tp.data_ptr(), n, int(pdt == torch.bfloat16), out.data_ptr(), elems, 7,
                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(out, _rank_order_sum(parts))
    assert L.b200q_sum_to_bf16(tp.data_ptr(), n, 1, out.data_ptr(), elems + 4, 7, None) == 1      # refused: elems % 8


def test_reduce_scatter_one_rank_world():
    """world = 1 through the per-rank entry point: the rank's own partial, rounded once."""
    import cudaop_b200 as ops
    L = ops.lib()
    elems = 8 * 4099
    part = torch.randn(elems, device="cuda")
    out = torch.zeros(elems, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(L.b200q_allreduce_signal_bytes() // 4, dtype=torch.int32, device="cuda")
    tp, to, tf = _ptr_table([part]), _ptr_table([out]), _ptr_table([flags])
    rc = L.b200q_reduce_scatter_to_bf16(tp.data_ptr(), to.data_ptr(), tf.data_ptr(), None, 0, 0, elems, 0, 1, 1, 0, 4,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert torch.equal(out, part.to(torch.bfloat16))


@pytest.mark.parametrize("pdt", [torch.bfloat16, torch.float32])
def test_fused_down_projection_allreduce_all_ranks_in_one_launch(pdt):
    import cudaop_b200 as ops
    L = ops.lib()
    world, M, N, K = 2, 1200, 512, 512                        # 10 tile rows: three row groups, ragged last
    rng = np.random.default_rng(5)
    A = [dev(oracle.encode_e4m3(rng.standard_normal((M, K), dtype=np.float32))) for _ in range(world)]
    B = [dev(oracle.encode_e4m3(rng.standard_normal((N, K), dtype=np.float32))) for _ in range(world)]
    rs = [dev(rng.uniform(0.5, 2.0, M).astype(np.float32)) for _ in range(world)]
    cs = dev(rng.uniform(0.001, 0.01, N).astype(np.float32))
    parts = [torch.zeros((M, N), dtype=pdt, device="cuda") for _ in range(world)]
    outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    counters = [torch.zeros(L.b200q_fused_allreduce_counter_bytes() // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(L.b200q_fused_allreduce_flag_bytes() // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    tp, to, tf = _ptr_table(parts), _ptr_table(outs), _ptr_table(flags)
    hA, hB, hrs, hp, hc = _host_table(A), _host_table(B), _host_table(rs), _host_table(parts), _host_table(counters)
    st = torch.cuda.current_stream().cuda_stream
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for epoch in (1, 2):
        for o in outs:
            o.fill_(float("nan"))
        rc = L.b200q_gemm_fp8_rowcol_allreduce_one_device(hA, hB, hrs, cs.data_ptr(), hp, hc, tp.data_ptr(), to.data_ptr(),
                                                          tf.data_ptr(), M, N, K, int(pdt == torch.bfloat16), 0, epoch,
                                                          world, min(20, sms // world), st)
        assert rc == 0
        torch.cuda.synchronize()
        assert ops.status() == 0
        want = _rank_order_sum(parts)                         # of the partial tiles the kernel itself wrote
        for o in outs:
            assert torch.equal(o, want)
    # and the partial tiles are the stand-alone down projection of each rank
    for r in range(world):
        ref = ops.gemm_fp8_rowcol(A[r], B[r], rs[r], cs, out_dtype=pdt)
        torch.testing.assert_close(parts[r].float(), ref.float(), rtol=2 ** -7, atol=1e-6)
    # ... which is right against the oracle
    a0 = oracle.decode_e4m3(A[0].cpu().numpy()); b0 = oracle.decode_e4m3(B[0].cpu().numpy())
    ref0 = oracle.gemm_f32(a0, b0, threads=8) * (rs[0].cpu().numpy()[:, None] * cs.cpu().numpy()[None, :])
    rep = oracle.error_report(parts[0].float().cpu().numpy() if pdt == torch.bfloat16
                              else oracle.decode_bf16(oracle.encode_bf16(parts[0].cpu().numpy())), ref0, k_dim=K)
    assert rep["rel_fro"] <= 1e-3 and rep["max_ulp_floor"] <= 2.0, rep


def test_a_wait_that_runs_out_sets_the_status_word_and_leaves_the_context_usable():
    """Rank 0 of a two-rank world calls the all-reduce; "rank 1" never does, so its flag is never raised.
    With a 5 ms limit the kernel gives up, records site 16 (the start barrier) and returns."""
    import cudaop_b200 as ops
    L = ops.lib()
    world, elems = 2, 8 * 2 * 64
    parts = [torch.ones(elems, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    outs = [torch.zeros(elems, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(L.b200q_allreduce_signal_bytes() // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    tp, to, tf = _ptr_table(parts), _ptr_table(outs), _ptr_table(flags)
    torch.cuda.synchronize()
    assert ops.status() == 0
    ops.set_wait_limit_ms(5, cross_rank=True)
    try:
        rc = L.b200q_allreduce_to_bf16(tp.data_ptr(), to.data_ptr(), tf.data_ptr(), None, None, 1, 0, elems, 0, world,
                                       1, 0, 2, torch.cuda.current_stream().cuda_stream)
        assert rc == 0                                         # the launch itself is fine
        torch.cuda.synchronize()                               # returns: the kernel gave up, it did not hang
        word = ops.status(clear=False)
        assert word & 0x80000000 and (word >> 24) & 0x7F == 16, hex(word)
        with pytest.raises(ops.WaitTimeout):
            ops.check_status("all-reduce")                     # the Python layer turns it into an exception
        assert ops.status() == 0                               # ... and cleared the word
    finally:
        ops.set_wait_limit_ms(10000, cross_rank=True)
    # the context is intact: an ordinary GEMM runs and is right
    aq, bq, sa, sb = oracle.make_fp8_case(128, 128, 128, seed=3)
    out = ops.gemm_fp8(dev(aq), dev(bq), sa, sb).float().cpu().numpy()
    ref = oracle.gemm_f32(oracle.decode_e4m3(aq) * np.float32(sa), oracle.decode_e4m3(bq) * np.float32(sb))
    rep = oracle.error_report(out, ref, k_dim=128)
    assert rep["rel_fro"] <= 1e-3 and ops.status() == 0
