// INT4 weight-only GEMM for decode shapes on warp-level mma.sync (the default of b200q_gemm_w4a16 for
// two tokens and more; one token goes to the CUDA-core kernel in gemm_w4a16_gemv.cu, and the tcgen05
// kernel in gemm_w4a16_tc.cu is selectable with b200q_w4a16_set_impl(1)):
//   Y[M,N] (bf16) = X[M,K] (bf16) * dequant(Wq)[N,K]^T,  w[n,k] = q[n,k] * S[n, k/128]
// Wq packs two signed 4-bit weights per byte along K, low nibble = lower K index
// (op/test/arch_primitives/ptx_mma_integer.cu:93-108); S is fp16, one scale per 128 K, no zero point.
//
// The operation is bound by reading Wq once from HBM (K*N/2 bytes), so the design is
// about keeping every weight byte in flight at once and doing exact arithmetic:
//   * a CTA owns 32 output columns and all of K; each of its 16 warps owns K-groups
//     g = w, w+16, ...; a lane reads 16 bytes (32 weights) of 4 rows per group with
//     streaming loads, next group's weights prefetched in registers;
//   * nibbles become bf16 integers in registers (exact: -8..7), activations stay bf16, the
//     product runs on mma.sync.m16n8k16 with fp32 accumulation (the tensor pipe is idle in a
//     bandwidth-bound kernel; the tcgen05 path would need the weights staged through shared
//     memory for no gain);
//   * the fp16 group scale multiplies the fp32 partial sum of its 128-K group, so no rounding
//     of q*s ever happens;
//   * the 16 warps' partials are summed in a fixed order through shared memory: deterministic.
// The MMA contraction index is a dummy, so the K order inside a 16-wide MMA step is permuted
// (the same way for both operands) to match the nibble order a 32-bit word yields.
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace w4a16 {

using ptx::mma_bf16_16816;

constexpr int kGroup = 128;
constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kColsPerCta = 32;


// nibbles (i, i+4) of a word, already offset to unsigned, -> two bf16 integers in [-8, 7]
__device__ __forceinline__ uint32_t nib_pair_to_bf16(uint32_t w_unsigned, int shift)
{
    const uint32_t v = ((w_unsigned >> shift) & 0x000F000Fu) | 0x43004300u;    // 128 + u
    __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v);
    const uint32_t c = 0x43084308u;                                            // 136
    b = __hsub2(b, *reinterpret_cast<const __nv_bfloat162*>(&c));
    return *reinterpret_cast<uint32_t*>(&b);
}

__global__ void __launch_bounds__(kThreads, 1)
w4a16_kernel(const __nv_bfloat16* __restrict__ X, const uint8_t* __restrict__ Wq, const __half* __restrict__ S,
             __nv_bfloat16* __restrict__ Y, int M, int N, int K)
{
    __shared__ float red[kWarps][16][kColsPerCta];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * kColsPerCta;
    const int m0 = blockIdx.y * 16;
    const int G = K / kGroup;
    const size_t wrow = static_cast<size_t>(K) / 2;

    float total[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) total[j][i] = 0.0f;

    auto load_w = [&](uint4 (&w)[4], int g) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + 8 * j + r;
            if (n < N) w[j] = ptx::ld_stream_v4(Wq + n * wrow + (g * kGroup + 32 * t) / 2);
            else w[j] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);   // zeros
        }
    };

    uint4 wcur[4], wnext[4];
    if (warp < G) load_w(wcur, warp);
    const bool row_lo = (m0 + r) < M, row_hi = (m0 + r + 8) < M;

    for (int g = warp; g < G; g += kWarps) {
        const bool more = (g + kWarps) < G;
        if (more) load_w(wnext, g + kWarps);

        uint4 xlo[4], xhi[4];
        const uint4* xl = reinterpret_cast<const uint4*>(X + static_cast<size_t>(m0 + r) * K + g * kGroup + 32 * t);
        const uint4* xh = reinterpret_cast<const uint4*>(X + static_cast<size_t>(m0 + r + 8) * K + g * kGroup + 32 * t);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            xlo[q] = row_lo ? __ldg(xl + q) : make_uint4(0, 0, 0, 0);
            xhi[q] = row_hi ? __ldg(xh + q) : make_uint4(0, 0, 0, 0);
        }
        float sc[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int n = n0 + 8 * j + 2 * t + c;
                sc[j][c] = (n < N) ? __half2float(__ldg(S + static_cast<size_t>(n) * G + g)) : 0.0f;
            }

        float acc[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;

#pragma unroll
        for (int q = 0; q < 4; ++q) {
            // activations of word q: (e0,e1) (e2,e3) (e4,e5) (e6,e7); MMA step 0 contracts
            // slots {e0,e4,e1,e5}, step 1 contracts {e2,e6,e3,e7}
            const uint32_t a0_0 = __byte_perm(xlo[q].x, xlo[q].z, 0x5410), a2_0 = __byte_perm(xlo[q].x, xlo[q].z, 0x7632);
            const uint32_t a1_0 = __byte_perm(xhi[q].x, xhi[q].z, 0x5410), a3_0 = __byte_perm(xhi[q].x, xhi[q].z, 0x7632);
            const uint32_t a0_1 = __byte_perm(xlo[q].y, xlo[q].w, 0x5410), a2_1 = __byte_perm(xlo[q].y, xlo[q].w, 0x7632);
            const uint32_t a1_1 = __byte_perm(xhi[q].y, xhi[q].w, 0x5410), a3_1 = __byte_perm(xhi[q].y, xhi[q].w, 0x7632);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t word = (q == 0 ? wcur[j].x : q == 1 ? wcur[j].y : q == 2 ? wcur[j].z : wcur[j].w) ^ 0x88888888u;
                const uint32_t v0 = nib_pair_to_bf16(word, 0), v1 = nib_pair_to_bf16(word, 4);
                const uint32_t v2 = nib_pair_to_bf16(word, 8), v3 = nib_pair_to_bf16(word, 12);
                mma_bf16_16816(acc[j], a0_0, a1_0, a2_0, a3_0, v0, v1);
                mma_bf16_16816(acc[j], a0_1, a1_1, a2_1, a3_1, v2, v3);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            total[j][0] = fmaf(acc[j][0], sc[j][0], total[j][0]);
            total[j][1] = fmaf(acc[j][1], sc[j][1], total[j][1]);
            total[j][2] = fmaf(acc[j][2], sc[j][0], total[j][2]);
            total[j][3] = fmaf(acc[j][3], sc[j][1], total[j][3]);
        }
        if (more) {
#pragma unroll
            for (int j = 0; j < 4; ++j) wcur[j] = wnext[j];
        }
    }

#pragma unroll
    for (int j = 0; j < 4; ++j) {
        red[warp][r][8 * j + 2 * t] = total[j][0];
        red[warp][r][8 * j + 2 * t + 1] = total[j][1];
        red[warp][r + 8][8 * j + 2 * t] = total[j][2];
        red[warp][r + 8][8 * j + 2 * t + 1] = total[j][3];
    }
    __syncthreads();
    {
        const int m = threadIdx.x >> 5, n = threadIdx.x & 31;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) s += red[w][m][n];
        if (m0 + m < M && n0 + n < N) Y[static_cast<size_t>(m0 + m) * N + n0 + n] = __float2bfloat16_rn(s);
    }
}

}  // namespace w4a16
}  // namespace b200q

extern "C" int b200q_gemm_w4a16_warp_mma(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K,
                                         int group, void* stream)
{
    using namespace b200q;
    if (X == nullptr || Wq == nullptr || S == nullptr || Y == nullptr) return cudaErrorInvalidValue;
    if (M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
    if (group != w4a16::kGroup || K % w4a16::kGroup != 0) return cudaErrorInvalidValue;
    if (!aligned16(X) || !aligned16(Wq)) return cudaErrorInvalidValue;
    dim3 grid((N + w4a16::kColsPerCta - 1) / w4a16::kColsPerCta, (M + 15) / 16);
    w4a16::w4a16_kernel<<<grid, w4a16::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(X), static_cast<const uint8_t*>(Wq), static_cast<const __half*>(S),
        static_cast<__nv_bfloat16*>(Y), M, N, K);
    return cudaGetLastError();
}
