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
