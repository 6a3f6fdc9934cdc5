"""The NVSwitch all-reduce kernel and the sharded MLP on 2, 4 and 8 real GPUs (each world size is skipped
when fewer GPUs are visible).  One process per GPU, NCCL only for the rendezvous; no rank is ever killed
or left waiting."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _need(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")


def _worker(rank, world, port, mode, pdt, out_dir):
    import torch.distributed as dist
    import cudaop_b200 as ops
    from cudaop_b200.mlp import TensorParallelMLP
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    T, H, I = 1200, 512, 1024           # 10 tile rows: three row groups in the fused kernel, ragged last
    # (1200 * 512 elements and 1024 intermediate features divide by 8 * world for 2, 4 and 8 ranks)
    case = oracle.make_mlp_case(T, H, I, seed=31)
    ts = [torch.from_numpy(np.ascontiguousarray(t)) for t in case[1:]]
    comm = {"multicast": "symm", "p2p": "symm", "nccl": "nccl", "fused": "fused", "fused_p2p": "fused",
            "pipelined": "pipelined", "pipelined_mc": "pipelined",
            "pipelined_ce": "pipelined_ce", "pipelined_ce_mc": "pipelined_ce", "pipelined_copy": "pipelined_copy"}[mode]
    pdtype = torch.bfloat16 if pdt == "bf16" else torch.float32
    mlp = TensorParallelMLP(*ts, rank=rank, world=world, max_tokens=T, chunks=2, comm=comm, partial_dtype=pdtype,
                            use_multicast=mode in ("multicast", "fused", "pipelined_mc", "pipelined_ce_mc"))
    x = torch.from_numpy(case[0].view(np.int16)).cuda().view(torch.bfloat16)
    y = mlp(x); mlp.wait(); y = y.clone()
    y2 = mlp(x); mlp.wait(); y2 = y2.clone()   # a second pass reuses (or alternates) buffers and flags
    y3 = mlp(x); mlp.wait()
    assert torch.equal(y3, y)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert torch.equal(y, y2)
    # the host-fed pipeline on top of the same layer: this rank's rows of the result arrive in pinned memory
    from cudaop_b200.mlp import HostFedMLP
    fed = HostFedMLP(mlp, T)
    x_host = x.cpu().pin_memory()
    y_host = torch.zeros((T, H), dtype=torch.bfloat16).pin_memory()
    for _ in range(3):
        fed.step(x_host, y_host)
    fed.finish(); torch.cuda.synchronize()
    assert ops.status() == 0
    assert torch.equal(y_host[fed.lo:fed.hi], y[fed.lo:fed.hi].cpu())
    # the kernel's sum against the fp32 partials of both ranks gathered with NCCL
    if mode == "nccl":
        # NCCL reduced mlp.partial in place: rebuild this rank's own partial with the stand-alone down projection
        mine = ops.gemm_fp8_rowcol(mlp.hq[:T], mlp.wd, mlp.shs[:T], mlp.sd, out_dtype=torch.float32)
    else:
        mine = mlp.partial[:T].contiguous()
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:                                    # fp32 sum in rank order, one rounding
        acc += p.float()
    want = acc.to(torch.bfloat16)
    torch.save({"y": y.cpu(), "want": want.cpu(), "comm": mlp.comm, "mc": getattr(mlp, "multicast", None)},
               os.path.join(out_dir, f"{mode}_{pdt}_r{rank}.pt"))
    dist.barrier(); dist.destroy_process_group()


MODES = ["pipelined", "pipelined_mc", "fused", "fused_p2p", "multicast", "p2p", "nccl", "pipelined_ce", "pipelined_ce_mc", "pipelined_copy"]


# two ranks: every transport and both partial types; four and eight ranks: the modes the benchmark times
# (side-stream all-reduce through the switch / by peer loads, and the fused latency mode) on bf16 partials
CASES = [(2, m, d) for m in MODES for d in ("bf16", "fp32")] + \
        [(w, m, "bf16") for w in (4, 8) for m in ("pipelined_mc", "pipelined", "fused", "pipelined_ce_mc", "pipelined_ce", "pipelined_copy")]


@pytest.mark.parametrize("world,mode,pdt", CASES)
def test_mlp_allreduce_across_ranks(world, mode, pdt, tmp_path):
    _need(world)
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 1000) + 20 * MODES.index(mode) + (10 if pdt == "fp32" else 0) + world
    mp.spawn(_worker, args=(world, port, mode, pdt, str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"{mode}_{pdt}_r{r}.pt") for r in range(world)]
    r0 = res[0]
    print(mode, "world:", world, "comm:", r0["comm"], "multicast:", r0["mc"])
    for r in res[1:]:
        assert torch.equal(r0["y"], r["y"])             # replicas bit-identical (nccl_mlp_test.cu:646-664)
    exact = (r0["y"] == r0["want"]).float().mean().item()
    if not r0["mc"] and mode != "nccl":
        # plain peer loads: fp32 sum in rank order, one rounding -- bit for bit
        assert torch.equal(r0["y"], r0["want"])
    else:
        # one rounding of the fp32 sum, but the switch (or NCCL's ring) adds in another order than rank order,
        # and the switch rounds the bf16 form itself: at most one bf16 ulp from the rank-order sum
        y, w = r0["y"].float(), r0["want"].float()
        ulp = torch.maximum(w.abs(), torch.full_like(w, 2.0 ** -120)).log2().floor().exp2() * 2.0 ** -7
        floor = 2.0 ** -8 * w.abs().max()               # sums that cancel: judged on the scale of the summands
        assert ((y - w).abs() <= torch.maximum(ulp, floor)).all()
        assert exact > (0.99 if pdt == "fp32" else 0.7), exact
