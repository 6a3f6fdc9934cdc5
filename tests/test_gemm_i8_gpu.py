"""Exact INT8 GEMM on the tensor cores (tcgen05 kind::i8): D = A * B^T + C in 32-bit integers.
Known answer and operand formulas: the S8 case of op/test/arch_primitives/ptx_mma_integer.cu:50-74,387-401."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, c=None):
    d = a.astype(np.int64) @ b.astype(np.int64).T
    if c is not None:
        d = d + c.astype(np.int64)
    return (d & 0xFFFFFFFF).astype(np.uint32).view(np.int32)          # 32-bit wrapping, as the hardware accumulates


def test_reference_coordinate_formulas_one_tile_with_accumulator():
    import cudaop_b200 as ops
    M, N, K = 16, 8, 32                                              # the reference's m16n8k32 tile
    r, c, k = np.arange(M)[:, None], np.arange(N)[:, None], np.arange(K)[None, :]
    a = (((r * 3 + k * 5 + 1) % 11) - 5).astype(np.int8)             # matrix_a_s8_value(row, inner)
    b = (((k * 7 + c * 2 + 3) % 9) - 4).astype(np.int8)              # matrix_b_s8_value(inner, column), stored [N, K]
    acc = (np.arange(M)[:, None] * 13 - np.arange(N)[None, :] * 5 - 37).astype(np.int32)
    d = ops.gemm_i8(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), torch.from_numpy(acc).cuda())
    torch.cuda.synchronize()
    assert np.array_equal(d.cpu().numpy(), _ref(a, b, acc))
    assert ops.status() == 0


@pytest.mark.parametrize("shape", [(128, 128, 128), (300, 520, 1040), (1, 8, 16), (513, 257, 4096), (2048, 2048, 2048)])
@pytest.mark.parametrize("pair", [1, 0])
def test_random_full_range_operands_are_exact(shape, pair):
    import cudaop_b200 as ops
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (N, K), dtype=np.int8)
    c = rng.integers(-2 ** 31, 2 ** 31, (M, N), dtype=np.int64).astype(np.int32) if M < 1000 else None
    ops.lib().b200q_fp8_set_2cta(pair)
    try:
        d = ops.gemm_i8(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), None if c is None else torch.from_numpy(c).cuda())
        torch.cuda.synchronize()
    finally:
        ops.lib().b200q_fp8_set_2cta(1)
    assert ops.status() == 0
    assert np.array_equal(d.cpu().numpy(), _ref(a, b, c))


def test_extreme_values_do_not_saturate():
    import cudaop_b200 as ops
    M, N, K = 128, 128, 8192
    a = np.full((M, K), -128, np.int8); b = np.full((N, K), -128, np.int8)
    d = ops.gemm_i8(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
    torch.cuda.synchronize()
    assert (d.cpu().numpy() == 128 * 128 * K).all()                  # 2^27: far from wrapping, must not clamp
    with pytest.raises(ValueError):
        ops.gemm_i8(torch.from_numpy(a).cuda().view(torch.uint8), torch.from_numpy(b).cuda())
    torch.cuda.synchronize()
