// Activation quantiser: bf16 rows -> E4M3 bytes + one fp32 scale per row (token).
//   s[r] = max|x[r,:]| / 448  (1.0 for an all-zero row),  q = e4m3_rn_satfinite(x * (1 / s[r]))
// (one IEEE reciprocal per row, one rounded product per element: a division per element made the
// kernel ALU-bound)
// Bandwidth-bound: one CTA per row, 16-byte streaming loads held in registers across the two
// passes (row maximum by warp shuffles + shared memory, then convert), 8 bytes written per 8 inputs.
// The CTA is sized to the row (64 to 256 threads, 8 to 14 vectors each): a row passes through three
// phases (load, reduce, convert + store) and only the first keeps memory busy, so short rows get small
// CTAs, many of which are resident per SM in different phases.
#include "common.cuh"
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include "../../include/b200q.h"

namespace b200q {
namespace quant {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ uint32_t cvt4_e4m3(float a, float b, float c, float d)
{
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// One CTA per row.  Every thread keeps its share of the row (up to kCache 16-byte vectors) in registers
// between the maximum pass and the convert pass, so a row is read from memory once; all of a thread's
// loads are issued before the first is used.  Rows longer than kThreads * kCache vectors re-read the rest.
template <int kThreads, int kCache, int kMinCtas>
__global__ void __launch_bounds__(kThreads, kMinCtas)
quant_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ X, uint8_t* __restrict__ Q, float* __restrict__ S, int rows,
                       int cols)
{
    __shared__ float wmax[kThreads / 32];
    __shared__ float s_scale;
    const int vecs = cols / 8;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4* x = reinterpret_cast<const uint4*>(X + static_cast<size_t>(row) * cols);
        uint4 cache[kCache];
#pragma unroll
        for (int i = 0; i < kCache; ++i) {
            const int v = threadIdx.x + i * kThreads;
            cache[i] = (v < vecs) ? __ldg(x + v) : make_uint4(0, 0, 0, 0);
        }
        float mx = 0.0f;
#pragma unroll
        for (int i = 0; i < kCache; ++i) {
            const uint32_t w[4] = {cache[i].x, cache[i].y, cache[i].z, cache[i].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) mx = fmaxf(mx, fmaxf(fabsf(bf16_lo(w[k])), fabsf(bf16_hi(w[k]))));
        }
        for (int v = threadIdx.x + kCache * kThreads; v < vecs; v += kThreads) {      // rows longer than the cache
            const uint4 u = __ldg(x + v);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) mx = fmaxf(mx, fmaxf(fabsf(bf16_lo(w[k])), fabsf(bf16_hi(w[k]))));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = mx;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = 0.0f;
            for (int i = 0; i < kThreads / 32; ++i) m = fmaxf(m, wmax[i]);
            // floor at the smallest normal float: the reciprocal below stays finite for rows of subnormal magnitudes
            const float sc = m > 0.0f ? fmaxf(__fdiv_rn(m, 448.0f), 1.17549435e-38f) : 1.0f;
            s_scale = sc;
            S[row] = sc;
        }
        __syncthreads();
        const float inv = __frcp_rn(s_scale);
        uint2* q = reinterpret_cast<uint2*>(Q + static_cast<size_t>(row) * cols);
        auto convert = [&](uint4 u) {
            uint2 o;
            o.x = cvt4_e4m3(__fmul_rn(bf16_lo(u.x), inv), __fmul_rn(bf16_hi(u.x), inv), __fmul_rn(bf16_lo(u.y), inv),
                            __fmul_rn(bf16_hi(u.y), inv));
            o.y = cvt4_e4m3(__fmul_rn(bf16_lo(u.z), inv), __fmul_rn(bf16_hi(u.z), inv), __fmul_rn(bf16_lo(u.w), inv),
                            __fmul_rn(bf16_hi(u.w), inv));
            return o;
        };
#pragma unroll
        for (int i = 0; i < kCache; ++i) {
            const int v = threadIdx.x + i * kThreads;
            if (v < vecs) q[v] = convert(cache[i]);
        }
        for (int v = threadIdx.x + kCache * kThreads; v < vecs; v += kThreads) q[v] = convert(__ldg(x + v));
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------------------
// bf16 rows -> NVFP4: packed E2M1 [rows, cols/2] + one UE4M3 scale per 16 K, written straight into the blocked
// layout the block-scaled GEMM reads (512-byte blocks of 128 rows x 4 scales, see b200q_nvfp4_swizzle_sf).
// Rule (the reference has formats only, op/test/arch_primitives/ptx_mma_fp4.cu:55-65,120-144,293-309):
//   sf = ue4m3_rn((max|blk| / 6) / g),  d = decode(sf) * g,  q = e2m1_rn(x * (1 / d)), all-zero where d < FLT_MIN.
// Bandwidth-bound (2 bytes read, 0.5625 written per element).  A warp takes 32 consecutive 64-element chunks of
// the flattened matrix; lane l's i-th 16-byte load is vector i * 32 + l of that span, so every load instruction
// reads 512 contiguous bytes.  A 16-element block lies in two neighbouring lanes (one shuffle for its maximum),
// the four scales of a 64-element chunk in eight lanes (three shuffles gather them into the one 32-bit word the
// blocked layout keeps them in).
__device__ __forceinline__ uint32_t cvt8_e2m1(const float (&y)[8])
{
    uint32_t out = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        out |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(make_float2(y[2 * i], y[2 * i + 1]), __NV_E2M1, cudaRoundNearest)) << (8 * i);
    return out;
}

__global__ void __launch_bounds__(256)
quant_rows_nvfp4_kernel(const __nv_bfloat16* __restrict__ X, uint32_t* __restrict__ Q, uint32_t* __restrict__ SF, int rows,
                        int cols, float g)
{
    const int lane = threadIdx.x & 31;
    const int c64 = cols / 64;                                        // 64-element chunks (= 512-byte scale blocks) per row
    const long long vecs = static_cast<long long>(rows) * cols / 8;   // 16-byte input vectors
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    const long long spans = (vecs + 255) / 256;                       // a warp's span: 256 vectors = 32 chunks
    const uint4* x = reinterpret_cast<const uint4*>(X);
    for (long long sp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; sp < spans; sp += warps) {
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const long long vi = sp * 256 + i * 32 + lane;
            v[i] = vi < vecs ? __ldg(x + vi) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const long long vi = sp * 256 + i * 32 + lane;
            const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
            float f[8];
            float mx = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                f[2 * k] = bf16_lo(w[k]); f[2 * k + 1] = bf16_hi(w[k]);
                mx = fmaxf(mx, fmaxf(fabsf(f[2 * k]), fabsf(f[2 * k + 1])));
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));      // the block's other half
            const float t = __fdiv_rn(__fdiv_rn(mx, 6.0f), g);
            const uint32_t s8 = (t > 0.0f) ? static_cast<uint32_t>(__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3)) : 0u;
            const float d = __fmul_rn(__half2float(__half(__nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(s8), __NV_E4M3))), g);
            const bool live = d >= 1.17549435e-38f;
            const float inv = live ? __frcp_rn(d) : 0.0f;
            float y[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) y[k] = __fmul_rn(f[k], inv);
            const uint32_t q = live ? cvt8_e2m1(y) : 0u;
            if (vi < vecs) Q[vi] = q;                                 // 8 elements -> 4 bytes, same order as the input
            // scales of the chunk: lanes 8j, 8j+2, 8j+4, 8j+6 hold blocks 0..3 of chunk (sp * 32 + i * 4 + j)
            uint32_t word = s8;
            word |= __shfl_down_sync(0xffffffffu, s8, 2) << 8;
            word |= __shfl_down_sync(0xffffffffu, s8, 4) << 16;
            word |= __shfl_down_sync(0xffffffffu, s8, 6) << 24;
            if ((lane & 7) == 0 && vi < vecs) {
                const long long chunk = vi >> 3;
                const int r = static_cast<int>(chunk / c64), j = static_cast<int>(chunk - static_cast<long long>(r) * c64);
                const size_t blk = static_cast<size_t>(r >> 7) * c64 + j;
                SF[blk * 128 + (r & 31) * 4 + ((r >> 5) & 3)] = word;
            }
        }
    }
    // scale words of the rows that pad the last 128-row block: zero
    const int pad_rows = ((rows + 127) / 128) * 128 - rows;
    const long long pad_words = static_cast<long long>(pad_rows) * c64;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < pad_words;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = rows + static_cast<int>(i / c64), j = static_cast<int>(i % c64);
        const size_t blk = static_cast<size_t>(r >> 7) * c64 + j;
        SF[blk * 128 + (r & 31) * 4 + ((r >> 5) & 3)] = 0u;
    }
}

}  // namespace quant
}  // namespace b200q

extern "C" int b200q_quant_rows_e4m3(const void* X, void* Q, float* S, int rows, int cols, void* stream)
{
    using namespace b200q;
    if (X == nullptr || Q == nullptr || S == nullptr) return cudaErrorInvalidValue;
    if (rows <= 0 || cols <= 0 || cols % 8 != 0) return cudaErrorInvalidValue;
    if (!aligned16(X) || (reinterpret_cast<uintptr_t>(Q) & 7u) != 0) return cudaErrorInvalidValue;
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(X);
    uint8_t* q = static_cast<uint8_t*>(Q);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int vecs = cols / 8;
    const int grid = rows < sms * 32 ? rows : sms * 32;
    if (vecs <= 64 * 8) quant::quant_rows_e4m3_kernel<64, 8, 12><<<grid, 64, 0, st>>>(x, q, S, rows, cols);
    else if (vecs <= 128 * 8) quant::quant_rows_e4m3_kernel<128, 8, 6><<<grid, 128, 0, st>>>(x, q, S, rows, cols);
    else if (vecs <= 256 * 8) quant::quant_rows_e4m3_kernel<256, 8, 3><<<grid, 256, 0, st>>>(x, q, S, rows, cols);
    else quant::quant_rows_e4m3_kernel<256, 14, 2><<<grid, 256, 0, st>>>(x, q, S, rows, cols);
    return cudaGetLastError();
}

extern "C" int b200q_quant_rows_nvfp4(const void* X, void* Q, void* SF_blocked, int rows, int cols, float global_scale, void* stream)
{
    using namespace b200q;
    if (X == nullptr || Q == nullptr || SF_blocked == nullptr) return cudaErrorInvalidValue;
    if (rows <= 0 || cols <= 0 || cols % 64 != 0 || !(global_scale > 0.0f)) return cudaErrorInvalidValue;
    if (!aligned16(X) || (reinterpret_cast<uintptr_t>(Q) & 3u) != 0 || !aligned16(SF_blocked)) return cudaErrorInvalidValue;
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const long long spans = (static_cast<long long>(rows) * cols / 8 + 255) / 256;
    long long blocks = (spans + 7) / 8;                    // 8 warps per CTA, one span per warp and pass
    if (blocks > sms * 8LL) blocks = sms * 8LL;
    if (blocks < 1) blocks = 1;
    quant::quant_rows_nvfp4_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(X), static_cast<uint32_t*>(Q), static_cast<uint32_t*>(SF_blocked), rows, cols, global_scale);
    return cudaGetLastError();
}
