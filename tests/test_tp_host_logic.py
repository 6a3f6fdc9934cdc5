"""Host-side logic of the tensor-parallel MLP on CPU: the sharding rule and a world-size-2
gloo all-reduce of per-rank partial results (the partials come from the oracle here — the CUDA
kernels are covered by the gpu-marked tests)."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from cudaop_b200.mlp import copy_exchange_plan, shard_mlp_weights


def test_shard_rule_matches_the_reference_layouts():
    # op/nccl/nccl_mlp_test.cu:321-352 in the [out, in] weight layout
    I, H, R = 12, 6, 4
    wg = torch.arange(I * H).reshape(I, H); wu = wg + 1000
    wd = torch.arange(H * I).reshape(H, I) + 5000
    sg = torch.arange(I).float(); su = sg + 100; sd = torch.arange(H).float()
    seen_rows, seen_cols = [], []
    for r in range(R):
        g, sgr, u, sur, d, sdr = shard_mlp_weights(wg, sg, wu, su, wd, sd, r, R)
        lo, hi = r * 3, (r + 1) * 3
        assert torch.equal(g, wg[lo:hi]) and torch.equal(u, wu[lo:hi]) and torch.equal(sgr, sg[lo:hi]) and torch.equal(sur, su[lo:hi])
        assert torch.equal(d, wd[:, lo:hi]) and d.is_contiguous() and torch.equal(sdr, sd)
        # the same split through the oracle's restatement of shard_a / shard_b on the transposed layouts
        assert np.array_equal(oracle.shard_cols(wg.numpy().T.copy(), r, R), g.numpy().T)
        assert np.array_equal(oracle.shard_rows(wd.numpy().T.copy(), r, R), d.numpy().T)
        seen_rows += list(range(lo, hi)); seen_cols += list(range(lo, hi))
    assert seen_rows == list(range(I)) and seen_cols == list(range(I))
    try:
        shard_mlp_weights(wg, sg, wu, su, wd, sd, 0, 5)
        assert False
    except ValueError:
        pass


def _rank_main(rank, world, port, case, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, wg, sg, wu, su, wd, sd = case
    g, sgr, u, sur, d, sdr = [t.numpy() for t in shard_mlp_weights(*[torch.from_numpy(a) for a in (wg, sg, wu, su, wd, sd)], rank, world)]
    X = oracle.decode_bf16(x)
    xq, sx = oracle.quant_rows_e4m3(X)
    Xd = oracle.decode_e4m3(xq)
    gg = oracle.gemm_f32(Xd, oracle.decode_e4m3(g)) * (sx[:, None] * sgr[None, :])
    uu = oracle.gemm_f32(Xd, oracle.decode_e4m3(u)) * (sx[:, None] * sur[None, :])
    h = oracle.decode_bf16(oracle.encode_bf16(oracle.swiglu(gg, uu)))
    hq, sh = oracle.quant_rows_e4m3(h)
    partial = torch.from_numpy(oracle.gemm_f32(oracle.decode_e4m3(hq), oracle.decode_e4m3(d)) * (sh[:, None] * sdr[None, :]))
    dist.all_reduce(partial, op=dist.ReduceOp.SUM)          # fp32 sum, every rank gets the same bits
    y = partial.to(torch.bfloat16)
    torch.save({"y": y, "h": torch.from_numpy(h)}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier(); dist.destroy_process_group()


def test_two_gloo_ranks_reduce_to_identical_replicas(tmp_path):
    T, H, I = 24, 64, 128
    case = oracle.make_mlp_case(T, H, I, seed=21)
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(2, port, case, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "r0.pt"); r1 = torch.load(tmp_path / "r1.pt")
    # replicas are bit-identical (op/nccl/nccl_mlp_test.cu:646-664 asserts rank0 == rank1)
    assert torch.equal(r0["y"], r1["y"])
    # sharded gate/up outputs are the column blocks of the un-sharded H
    x, wg, sg, wu, su, wd, sd = case
    X = oracle.decode_bf16(x); xq, sx = oracle.quant_rows_e4m3(X); Xd = oracle.decode_e4m3(xq)
    g = oracle.gemm_f32(Xd, oracle.decode_e4m3(wg)) * (sx[:, None] * sg[None, :])
    u = oracle.gemm_f32(Xd, oracle.decode_e4m3(wu)) * (sx[:, None] * su[None, :])
    h = oracle.decode_bf16(oracle.encode_bf16(oracle.swiglu(g, u)))
    assert np.array_equal(np.concatenate([r0["h"].numpy(), r1["h"].numpy()], axis=1), h)
    # and the reduced result is the un-sharded MLP to quantisation accuracy
    hq, sh = oracle.quant_rows_e4m3(h)
    y_full = oracle.gemm_f32(oracle.decode_e4m3(hq), oracle.decode_e4m3(wd)) * (sh[:, None] * sd[None, :])
    rel = np.linalg.norm(r0["y"].float().numpy() - y_full) / np.linalg.norm(y_full)
    assert rel < 3e-2, rel


def test_copy_exchange_plan_reproduces_the_rank_order_sum_on_every_rank():
    """The index plan of the copy-engine exchange, played on the host for 1, 2, 4 and 8 ranks: every rank ends
    with the fp32 rank-order sum rounded once, and at every step of the first phase the ranks read from
    pairwise different peers."""
    import pytest
    rng = np.random.default_rng(3)
    for world in (1, 2, 4, 8):
        n = 8 * world * 5
        partial = [torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(torch.bfloat16) for _ in range(world)]
        want = torch.zeros(n)
        for p in partial:
            want += p.float()
        want = want.to(torch.bfloat16)
        plans = [copy_exchange_plan(r, world, n) for r in range(world)]
        y = [torch.full((n,), float("nan"), dtype=torch.bfloat16) for _ in range(world)]
        for r, ((lo, hi), pulls, _) in enumerate(plans):
            staged = {peer: partial[peer][a:z].clone() for peer, a, z in pulls}
            assert all((a, z) == (lo, hi) for _, a, z in pulls) and sorted(staged) == [q for q in range(world) if q != r]
            acc = torch.zeros(hi - lo)
            for q in range(world):                        # rank order, the own part read in place
                acc += (partial[r][lo:hi] if q == r else staged[q]).float()
            y[r][lo:hi] = acc.to(torch.bfloat16)
        for r, (_, _, pulls) in enumerate(plans):
            for peer, a, z in pulls:
                assert (a, z) == plans[peer][0]           # a peer's own range, which that peer has summed
                y[r][a:z] = y[peer][a:z]
        for r in range(world):
            assert torch.equal(y[r], want)
        for step in range(world - 1):                     # no two ranks pull from the same peer at the same step
            assert len({plans[r][1][step][0] for r in range(world)}) == world
    with pytest.raises(ValueError):
        copy_exchange_plan(0, 3, 100)
    with pytest.raises(ValueError):
        copy_exchange_plan(2, 2, 32)
