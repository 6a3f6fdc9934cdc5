// INT4 weight-only GEMV for one to four tokens (decode), sm_100a, CUDA cores only:
//   Y[M,N] (bf16) = X[M,K] (bf16) * dequant(Wq)[N,K]^T,   w[n,k] = q[n,k] * S[n, k/128]
// Wq: two signed nibbles per byte along K, low nibble = lower K
// (op/test/arch_primitives/ptx_mma_integer.cu:93-108); S fp16, one per 128 K, no zero point.
//
// With so few tokens the tensor cores have nothing to offer (the warp-level MMA is throttled on this
// architecture, and a tcgen05 pipeline costs more in hand-offs than the arithmetic is worth): the
// operation is one pass over Wq, and the aim is to have every byte of it requested at once.
//   * A warp owns 4 weight rows x 1024 K: one 16-byte streaming load per lane and row, all four issued
//     before anything else, then the four fp16 group scales (a lane's 32 weights lie in one group).
//     A CTA is K/1024 such warps (at most 8, which then walk several slices; a few row blocks when K is
//     short); N/4 CTAs of 128 threads for K = 4096, all resident at once, so the whole matrix is in
//     flight after the first instruction.
//   * Only then the kernel waits for the previous kernel of the stream (griddepcontrol.wait; a no-op
//     without programmatic dependent launch) and reads its 32 activations per token.
//   * Nibble -> fp32 without shifts or conversions: (word & (0xF << 4i)) | bits(2^(23-4i)) is the float
//     2^(23-4i) + u exactly (u = nibble ^ 8 = q + 8), one subtraction gives q.  fp32 FMAs, the group
//     scale multiplies the lane's fp32 partial sum (q*s is never rounded), butterfly reduction over
//     the lanes, and the K slices of a row are added in a fixed order through shared memory.
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace w4gemv {

constexpr int kGroup = 128;
constexpr int kRows = 4;            // weight rows per warp
constexpr int kSliceK = 1024;       // K covered by one warp-wide 16-byte load
constexpr int kMaxSliceWarps = 8;  // longer K: a warp walks several slices

// nibble i (0..7) of `word` (already ^ 0x88888888, i.e. unsigned q + 8) as fp32 q
__device__ __forceinline__ void word_to_f32(uint32_t word, float (&f)[8])
{
    const uint32_t hi = word >> 12;       // nibbles 5, 6, 7 at bit positions 8, 12, 16
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int pos = (i < 5) ? 4 * i : 4 * (i - 3);            // bit position of the nibble in the word used
        const uint32_t src = (i < 5) ? word : hi;
        const uint32_t magic = static_cast<uint32_t>(127 + 23 - pos) << 23;       // 2^(23 - pos)
        const float bias = __uint_as_float(magic) + 8.0f;                        // exact: pos <= 16
        f[i] = __uint_as_float((src & (0xFu << pos)) | magic) - bias;
    }
}

template <int MT>
__global__ void __launch_bounds__(256)
w4a16_gemv_kernel(const __nv_bfloat16* __restrict__ X, const uint8_t* __restrict__ Wq, const __half* __restrict__ S,
                  __nv_bfloat16* __restrict__ Y, int M, int N, int K)
{
    extern __shared__ float red[];          // [row blocks][slice warps][kRows][MT]
    const int lane = threadIdx.x, ks = threadIdx.y, rb = threadIdx.z;
    const int slices = blockDim.y;          // warps that share a row block; warp ks takes K slices ks, ks + slices, ...
    const int n0 = (blockIdx.x * blockDim.z + rb) * kRows;
    const int m0 = blockIdx.y * MT;
    const int G = K / kGroup;

    auto load_w = [&](uint4 (&w)[kRows], float (&sc)[kRows], int k0) {
        const bool k_ok = k0 < K;                     // K % 128 == 0: a 32-weight chunk is entirely inside or outside
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int n = n0 + r;
            if (k_ok && n < N) w[r] = ptx::ld_stream_v4(Wq + static_cast<size_t>(n) * (K / 2) + k0 / 2);
            else w[r] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);    // q = 0
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int n = n0 + r;
            sc[r] = (k_ok && n < N) ? __half2float(__ldg(S + static_cast<size_t>(n) * G + k0 / kGroup)) : 0.0f;
        }
    };

    // 1. weights and scales of the first slice: nothing here depends on the kernel before this one
    uint4 w[kRows];
    float sc[kRows];
    int k0 = ks * kSliceK + lane * 32;                // this lane's 32 consecutive K (inside one scale group)
    load_w(w, sc, k0);

    // 2. let the next kernel of the stream start its own weight stream; wait for the previous one before X
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float acc[kRows][MT];
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

    for (; k0 < K; k0 += slices * kSliceK) {
        // 3. activations of this lane's K chunk
        float x[MT][32];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const bool ok = (m0 + m) < M;
            const uint4* src = reinterpret_cast<const uint4*>(X + static_cast<size_t>(ok ? m0 + m : 0) * K + k0);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 v = ok ? __ldg(src + q) : make_uint4(0, 0, 0, 0);
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    x[m][8 * q + 2 * e] = __uint_as_float(u[e] << 16);
                    x[m][8 * q + 2 * e + 1] = __uint_as_float(u[e] & 0xFFFF0000u);
                }
            }
        }
        // 4. dot products, fp32; the group scale multiplies the chunk's partial sum
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float part[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) part[m] = 0.0f;
            const uint32_t words[4] = {w[r].x ^ 0x88888888u, w[r].y ^ 0x88888888u, w[r].z ^ 0x88888888u, w[r].w ^ 0x88888888u};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float f[8];
                word_to_f32(words[q], f);
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int m = 0; m < MT; ++m) part[m] = fmaf(f[i], x[m][8 * q + i], part[m]);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = fmaf(part[m], sc[r], acc[r][m]);
        }
        if (k0 + slices * kSliceK < K) load_w(w, sc, k0 + slices * kSliceK);     // long K only: the next slice of this warp
    }

    // 5. over the lanes (each warp does this once), then over the K slices in a fixed order
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[r][m];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
            acc[r][m] = v;
        }
    float* mine = red + (static_cast<size_t>(rb) * slices + ks) * (kRows * MT);
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < kRows; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) mine[r * MT + m] = acc[r][m];
    }
    __syncthreads();
    if (ks == 0 && lane < kRows * MT) {
        const int r = lane / MT, m = lane % MT;
        float s = 0.0f;
        for (int j = 0; j < slices; ++j) s += red[(static_cast<size_t>(rb) * slices + j) * (kRows * MT) + lane];
        if (n0 + r < N && m0 + m < M) Y[static_cast<size_t>(m0 + m) * N + n0 + r] = __float2bfloat16_rn(s);
    }
}

}  // namespace w4gemv

// Called by b200q_gemm_w4a16 for M <= 4.  pdl: launch with programmatic stream serialisation, i.e. this
// kernel may start (and stream its weights) while the previous kernel of the stream is still running.
int gemm_w4a16_gemv(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int group, int pdl, void* stream)
{
    using namespace w4gemv;
    if (X == nullptr || Wq == nullptr || S == nullptr || Y == nullptr) return cudaErrorInvalidValue;
    if (M <= 0 || M > 4 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
    if (group != kGroup || K % kGroup != 0) return cudaErrorInvalidValue;
    if (!aligned16(X) || !aligned16(Wq)) return cudaErrorInvalidValue;
    const int all_slices = (K + kSliceK - 1) / kSliceK;
    const int slices = all_slices < kMaxSliceWarps ? all_slices : kMaxSliceWarps;     // warps per row block
    const int rbs = slices >= 4 ? 1 : 4 / slices;              // at least four warps per CTA
    const int mt = (M == 1) ? 1 : 2;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((N + rbs * kRows - 1) / (rbs * kRows), (M + mt - 1) / mt);
    cfg.blockDim = dim3(32, slices, rbs);
    cfg.dynamicSmemBytes = static_cast<size_t>(rbs) * slices * kRows * mt * sizeof(float);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(X);
    const uint8_t* wq = static_cast<const uint8_t*>(Wq);
    const __half* s = static_cast<const __half*>(S);
    __nv_bfloat16* y = static_cast<__nv_bfloat16*>(Y);
    if (mt == 1) return cudaLaunchKernelEx(&cfg, w4a16_gemv_kernel<1>, x, wq, s, y, M, N, K);
    return cudaLaunchKernelEx(&cfg, w4a16_gemv_kernel<2>, x, wq, s, y, M, N, K);
}

}  // namespace b200q
