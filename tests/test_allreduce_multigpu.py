"""The NVSwitch all-reduce kernel and the sharded MLP on 2 real GPUs (skipped with fewer).
One process per GPU, NCCL only for the rendezvous; no rank is ever killed or left waiting."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _need_two():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")


def _worker(rank, world, port, mode, pdt, out_dir):
    import torch.distributed as dist
    import cudaop_b200 as ops
    from cudaop_b200.mlp import TensorParallelMLP
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    T, H, I = 1200, 512, 1024           # 10 tile rows: three row groups in the fused kernel, ragged last
    case = oracle.make_mlp_case(T, H, I, seed=31)
    ts = [torch.from_numpy(np.ascontiguousarray(t)) for t in case[1:]]
    comm = {"multicast": "symm", "p2p": "symm", "nccl": "nccl", "fused": "fused", "fused_p2p": "fused",
            "pipelined": "pipelined"}[mode]
    pdtype = torch.bfloat16 if pdt == "bf16" else torch.float32
    mlp = TensorParallelMLP(*ts, rank=rank, world=world, max_tokens=T, chunks=2, comm=comm, partial_dtype=pdtype,
                            use_multicast=mode in ("multicast", "fused"))
    x = torch.from_numpy(case[0].view(np.int16)).cuda().view(torch.bfloat16)
    y = mlp(x); mlp.wait(); y = y.clone()
    y2 = mlp(x); mlp.wait(); y2 = y2.clone()   # a second pass reuses (or alternates) buffers and flags
    y3 = mlp(x); mlp.wait()
    assert torch.equal(y3, y)
    torch.cuda.synchronize()
    assert ops.status() == 0
    assert torch.equal(y, y2)
    # the kernel's sum against the fp32 partials of both ranks gathered with NCCL
    if mode == "nccl":
        want = mlp.partial.to(torch.bfloat16)          # NCCL reduced the partials in place
    else:
        parts = [torch.empty_like(mlp.partial) for _ in range(world)]
        dist.all_gather(parts, mlp.partial.contiguous())
        acc = torch.zeros_like(parts[0], dtype=torch.float32)
        for p in parts:                                # fp32 sum in rank order, one rounding
            acc += p.float()
        want = acc.to(torch.bfloat16)
    torch.save({"y": y.cpu(), "want": want.cpu(), "comm": mlp.comm, "mc": getattr(mlp, "multicast", None)},
               os.path.join(out_dir, f"{mode}_{pdt}_r{rank}.pt"))
    dist.barrier(); dist.destroy_process_group()


@pytest.mark.parametrize("pdt", ["bf16", "fp32"])
@pytest.mark.parametrize("mode", ["pipelined", "fused", "fused_p2p", "multicast", "p2p", "nccl"])
def test_two_rank_mlp_allreduce(mode, pdt, tmp_path):
    _need_two()
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 1000) + {"multicast": 0, "p2p": 1, "nccl": 2, "fused": 3, "fused_p2p": 4, "pipelined": 10}[mode] + (5 if pdt == "fp32" else 0)
    mp.spawn(_worker, args=(2, port, mode, pdt, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(tmp_path / f"{mode}_{pdt}_r0.pt"); r1 = torch.load(tmp_path / f"{mode}_{pdt}_r1.pt")
    print(mode, "comm:", r0["comm"], "multicast:", r0["mc"])
    assert torch.equal(r0["y"], r1["y"])                # replicas bit-identical (nccl_mlp_test.cu:646-664)
    if mode in ("nccl", "p2p", "fused_p2p", "pipelined"):
        # plain peer loads: fp32 sum in rank order, one rounding -- bit for bit
        assert torch.equal(r0["y"], r0["want"])
    else:
        # one rounding of the fp32 sum; the switch may add in a different order than rank order
        d = (r0["y"].float() - r0["want"].float()).abs().max().item()
        assert d <= 2.0 ** -7 * r0["want"].float().abs().max().item()
        assert (r0["y"] == r0["want"]).float().mean().item() > (0.99 if pdt == "fp32" else 0.7)
