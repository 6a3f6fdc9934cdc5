"""Parity of the SwiGLU MLP forward (quantise -> gate/up+SwiGLU -> quantise -> down) with the oracle."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import CORES, assert_bar, bf16_to_f32, dev

pytestmark = pytest.mark.gpu


def _oracle_chain(x_bf16, wg, sg, wu, su):
    X = oracle.decode_bf16(x_bf16)
    xq, sx = oracle.quant_rows_e4m3(X)
    Xd = oracle.decode_e4m3(xq)
    g = oracle.gemm_f32(Xd, oracle.decode_e4m3(wg), threads=CORES) * (sx[:, None] * sg[None, :])
    u = oracle.gemm_f32(Xd, oracle.decode_e4m3(wu), threads=CORES) * (sx[:, None] * su[None, :])
    return xq, sx, oracle.swiglu(g, u)


def _tensors(case):
    return [torch.from_numpy(np.ascontiguousarray(t)) for t in case[1:]]


@pytest.mark.parametrize("dims", [(192, 512, 1024), (130, 256, 384)])
def test_single_rank_forward_stage_by_stage(dims):
    from cudaop_b200.mlp import TensorParallelMLP
    import cudaop_b200 as ops
    T, H, I = dims
    case = oracle.make_mlp_case(T, H, I, seed=11)
    x, wg, sg, wu, su, wd, sd = case
    mlp = TensorParallelMLP(*_tensors(case), max_tokens=T)
    y = mlp(dev(x, torch.bfloat16))
    torch.cuda.synchronize()
    assert ops.status() == 0 and mlp.kernel_launches_per_forward == 4
    xq_ref, sx_ref, h_ref = _oracle_chain(x, wg, sg, wu, su)
    # 1. activation quantiser: bit exact
    assert np.array_equal(mlp.sx.cpu().numpy().view(np.uint32), sx_ref.view(np.uint32))
    xq = mlp.xq.cpu().numpy()
    assert ((xq == xq_ref) | (((xq | xq_ref) & 0x7F) == 0)).all()
    # 2. gate/up + SwiGLU against the oracle on the same quantised bytes
    h_gpu = mlp.h.view(torch.int16).cpu().numpy().view(np.uint16)
    assert_bar(oracle.decode_bf16(h_gpu), h_ref, H, "swiglu")
    # 3. second quantiser on the GPU's own H bytes: bit exact
    hq_ref, sh_ref = oracle.quant_rows_e4m3(oracle.decode_bf16(h_gpu))
    assert np.array_equal(mlp.shs.cpu().numpy().view(np.uint32), sh_ref.view(np.uint32))
    hq = mlp.hq.cpu().numpy()
    assert ((hq == hq_ref) | (((hq | hq_ref) & 0x7F) == 0)).all()
    # 4. down projection against the oracle fed the GPU's quantised H
    y_ref = oracle.gemm_f32(oracle.decode_e4m3(hq), oracle.decode_e4m3(wd), threads=CORES) * (sh_ref[:, None] * sd[None, :])
    assert_bar(bf16_to_f32(y), y_ref, I, "down")
    # information: distance to an MLP with unquantised activations (quantisation error, not kernel error)
    Xf = oracle.decode_bf16(x)
    gf = (Xf @ (oracle.decode_e4m3(wg) * sg[:, None]).T); uf = (Xf @ (oracle.decode_e4m3(wu) * su[:, None]).T)
    yf = oracle.swiglu(gf.astype(np.float32), uf.astype(np.float32)) @ (oracle.decode_e4m3(wd) * sd[:, None]).T
    e2e = np.linalg.norm(bf16_to_f32(y) - yf) / np.linalg.norm(yf)
    print("end-to-end distance to the fp32-activation MLP:", e2e)
    assert e2e < 0.1


@pytest.mark.parametrize("pdt", [torch.float32, torch.bfloat16])
def test_two_rank_shards_sum_to_the_single_rank_result(pdt):
    # op/nccl/nccl_mlp_test.cu:321-352: column-parallel then row-parallel shards; the sum of the
    # ranks' partial outputs is the un-sharded result.  Both ranks are run one after the other on
    # this GPU and their partials are added in fp32 in rank order, as the all-reduce does.
    from cudaop_b200.mlp import TensorParallelMLP
    T, H, I = 160, 256, 1024
    case = oracle.make_mlp_case(T, H, I, seed=12)
    x = dev(case[0], torch.bfloat16)
    full = TensorParallelMLP(*_tensors(case), max_tokens=T)
    y1 = full(x).float()
    acc = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    hs, ref_sum = [], np.zeros((T, H), np.float32)
    for r in range(2):
        # comm="nccl" only to get a rank object without a process group; that mode always keeps fp32 partials,
        # so the bf16 case gives the rank a bf16 partial buffer by hand (what the symmetric-memory modes hold)
        m = TensorParallelMLP(*_tensors(case), rank=r, world=2, max_tokens=T, comm="nccl", partial_dtype=pdt)
        assert m.partial_dtype == torch.float32
        m.partial_dtype = pdt
        m.partial = torch.empty((T, H), dtype=pdt, device="cuda")
        assert m.wg.shape == (I // 2, H) and m.wd.shape == (H, I // 2)
        m._stage(x, None, 0, T)
        torch.cuda.synchronize()
        acc += m.partial.float()
        hs.append(m.h.clone())
        # this rank's partial against the oracle on the rank's own quantised bytes
        hq = m.hq.cpu().numpy(); sh = m.shs.cpu().numpy()
        wd_r = case[5][:, r * (I // 2):(r + 1) * (I // 2)]
        ref_r = oracle.gemm_f32(oracle.decode_e4m3(hq), oracle.decode_e4m3(wd_r), threads=CORES) * (sh[:, None] * case[6][None, :])
        ref_sum += ref_r
        if pdt == torch.bfloat16:
            assert_bar(m.partial.float().cpu().numpy(), ref_r, I // 2, f"bf16 partial of rank {r}")
        else:
            np.testing.assert_allclose(m.partial.cpu().numpy(), ref_r, rtol=3e-5, atol=1e-6 * np.abs(ref_r).max())
    # the sharded gate/up outputs are exactly the column blocks of the un-sharded one
    assert torch.equal(torch.cat(hs, dim=1), full.h)
    y2 = acc.to(torch.bfloat16).float()
    # per-rank token scales differ from the single-rank ones, so H is quantised to E4M3 (3 mantissa
    # bits, ~2-3 % per element) on two different grids: the two results agree to that accuracy,
    # not bit for bit
    rel = ((y2 - y1).norm() / y1.norm()).item()
    assert rel < 5e-2, rel
    if pdt == torch.float32:
        # fp32 partials (the reference's ncclFloat contract): the reduced output meets the bar
        # against the oracle's sum; bf16 partials are a stage of their own, checked above
        assert_bar(y2.cpu().numpy(), ref_sum, I, "tp2 sum")


def test_prepare_quantises_the_next_batch_ahead_with_the_same_bits():
    """prepare(x) on the side stream, then forward(x): identical output to a forward that quantises by itself;
    the two slots alternate; a forward on a DIFFERENT tensor ignores the prepared batch."""
    from cudaop_b200.mlp import TensorParallelMLP
    import cudaop_b200 as ops
    T, H, I = 192, 512, 1024
    case = oracle.make_mlp_case(T, H, I, seed=13)
    mlp = TensorParallelMLP(*_tensors(case), max_tokens=T)
    x = dev(case[0], torch.bfloat16)
    y_plain = mlp(x).clone()
    for _ in range(5):                                  # more steps than slots
        mlp.prepare(x)
        y = mlp(x)
        assert mlp._prep is None                        # consumed
        torch.cuda.synchronize()
        assert torch.equal(y, y_plain)
    x2 = (x.float() * 0.5).to(torch.bfloat16)
    y2_plain = mlp(x2).clone()
    mlp.prepare(x)
    y2 = mlp(x2)                                        # another batch: quantised inside the forward
    torch.cuda.synchronize()
    assert torch.equal(y2, y2_plain) and mlp._prep is not None
    mlp.cancel_prepared()
    assert mlp._prep is None and ops.status() == 0


@pytest.mark.parametrize("prepare_ahead", [True, False])
def test_host_fed_pipeline_leaves_the_result_in_pinned_memory(prepare_ahead):
    """HostFedMLP on one rank: inputs from pinned host memory, double-buffered copies on their own streams, the result
    back in pinned memory -- the same bits as a device-resident forward, for more steps than buffers."""
    from cudaop_b200.mlp import HostFedMLP, TensorParallelMLP
    import cudaop_b200 as ops
    T, H, I = 192, 512, 1024
    case = oracle.make_mlp_case(T, H, I, seed=17)
    mlp = TensorParallelMLP(*_tensors(case), max_tokens=T)
    x = dev(case[0], torch.bfloat16)
    want = mlp(x).clone().cpu()
    fed = HostFedMLP(mlp, T, prepare_ahead=prepare_ahead)
    xs = [x.cpu().pin_memory(), (x.float() * 0.5).to(torch.bfloat16).cpu().pin_memory()]
    want2 = mlp(xs[1].cuda()).clone().cpu()
    y_host = [torch.zeros((T, H), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    for i in range(5):
        fed.step(xs[i & 1], y_host[i & 1])
    fed.finish(); torch.cuda.synchronize()
    assert ops.status() == 0
    assert torch.equal(y_host[0], want) and torch.equal(y_host[1], want2)
