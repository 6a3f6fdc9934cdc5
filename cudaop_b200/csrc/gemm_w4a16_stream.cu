// INT4 weight-only GEMV for one token (decode), sm_100a: the streaming form.
//   Y[1,N] (bf16) = X[1,K] (bf16) * dequant(Wq)[N,K]^T,   w[n,k] = q[n,k] * S[n, k/128]
// Wq: two signed nibbles per byte along K, low nibble = lower K
// (op/test/arch_primitives/ptx_mma_integer.cu:93-108); S fp16, one per 128 K, no zero point.
//
// A call moves N*K/2 bytes once and does almost nothing else, so what matters is that the memory system
// never idles between calls:
//   * one CTA per SM owns a contiguous block of rows (all of K) small enough — at most 56 KiB of weights —
//     that three CTAs fit in an SM's shared memory and registers;
//   * the first thing a CTA does is to issue plain bulk copies (cp.async.bulk, no multicast) of its whole
//     weight block and its scales, then to let the next kernel of the stream start
//     (griddepcontrol.launch_dependents); only then does it wait for the previous kernel
//     (griddepcontrol.wait) before it touches X or Y.  With programmatic dependent launch the CTAs of the
//     next one or two calls are therefore resident and streaming THEIR weights while this call computes;
//     without it both instructions are no-ops.  The previous kernel must not be the one that writes Wq or S.
//   * arithmetic is integer, as in the shared-memory GEMV of gemm_w4a16_gemv.cu but with the activation
//     conversion done once per CTA instead of once per eight rows: 256 threads turn X into 21-bit fixed
//     point relative to the largest exponent of each 64-element unit (exact for every bf16 within 2^13 of
//     that maximum, off by at most 2^-22 of it otherwise), split into three byte planes laid out in the
//     order in which a weight word falls apart into bytes; every thread then keeps the planes of its 64 K
//     in registers and walks the CTA's rows: per weight word two logic operations give (q + 8) as bytes,
//     six dp4a accumulate the exact 32-bit sums (in six independent chains), and once per row and unit the sum loses 8 * sum(x), is
//     converted and scaled by 2^-shift * S in fp32.  q * s is never rounded.
//   * the 16-byte shared-memory reads of the two halves of a thread's 32 weight bytes are ordered by lane so
//     that a quarter-warp touches eight different bank groups.
// Rows are reduced over their K/64 threads by warp shuffles and a fixed-order sum over warps: deterministic.
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace w4s {

using ptx::bulk_load;
using ptx::dp4a_us;
using ptx::dp4a_uu;
using ptx::max_nan;

constexpr int kGroup = 128;
constexpr int kThreads = 256;
constexpr int kUnit = 64;                 // K per thread in the main loop; one fixed-point exponent per unit
constexpr int kMaxRowsPerThread = 7;      // rows a thread walks: rows_per_cta / (kThreads / (K / 64)); 8 slots in the reduction
constexpr int kSlabBytes = 56 * 1024;     // weights of one CTA
constexpr int kCopyPiece = 16 * 1024;     // one bulk copy

struct Layout {                           // byte offsets inside dynamic shared memory
    int w, s, planes, inv, sumx, red, bar, total;
};
__host__ __device__ inline Layout layout(int K, int rows_per_cta)
{
    Layout L;
    L.w = 0;
    L.s = kSlabBytes;
    L.planes = L.s + ((rows_per_cta * (K / kGroup) * 2 + 127) & ~127);
    L.inv = L.planes + 3 * K;
    L.sumx = L.inv + (K / kUnit) * 4;
    L.red = L.sumx + (K / kUnit) * 4;
    L.bar = L.red + (kThreads / 32) * 8 * 4;
    L.total = L.bar + 16;
    return L;
}

__global__ void __launch_bounds__(kThreads, 3)
w4a16_stream_kernel(const __nv_bfloat16* __restrict__ X, const uint8_t* __restrict__ Wq, const __half* __restrict__ S,
                    __nv_bfloat16* __restrict__ Y, int N, int K, int rows_per_cta, int scales_by_copy, uint32_t* status)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = K / kGroup;
    const int U = K / kUnit;                        // threads that cover K once (a multiple of 32)
    const int RS = kThreads / U;                    // rows in flight per pass
    // rows split as evenly as possible over the grid: CTA b owns [b N / grid, (b + 1) N / grid), at most rows_per_cta rows
    const int n0 = static_cast<int>(static_cast<long long>(blockIdx.x) * N / gridDim.x);
    const int nrows = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * N / gridDim.x) - n0;
    const size_t row_bytes = static_cast<size_t>(K) / 2;
    const Layout L = layout(K, rows_per_cta);
    uint8_t* w_sm = smem + L.w;
    __half* s_sm = reinterpret_cast<__half*>(smem + L.s);
    uint8_t* planes = smem + L.planes;              // [3][K]
    float* inv_sm = reinterpret_cast<float*>(smem + L.inv);
    int* sumx_sm = reinterpret_cast<int*>(smem + L.sumx);
    float* red = reinterpret_cast<float*>(smem + L.red);
    const uint32_t bar = ptx::smem_u32(smem + L.bar);

    // 1. this CTA's weights (one contiguous block of memory) and scales: nothing here depends on the kernel before
    const uint32_t w_bytes = static_cast<uint32_t>(nrows * row_bytes);
    const uint32_t s_bytes = static_cast<uint32_t>(nrows) * G * 2;
    if (tid == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_mbar_init();
        ptx::mbar_arrive_expect_tx(bar, w_bytes + (scales_by_copy ? s_bytes : 0u));
        const uint8_t* src = Wq + static_cast<size_t>(n0) * row_bytes;
        for (uint32_t off = 0; off < w_bytes; off += kCopyPiece)
            bulk_load(ptx::smem_u32(w_sm) + off, src + off, min(static_cast<uint32_t>(kCopyPiece), w_bytes - off), bar);
        if (scales_by_copy) bulk_load(ptx::smem_u32(s_sm), S + static_cast<size_t>(n0) * G, s_bytes, bar);
    }
    if (!scales_by_copy)
        for (int i = tid; i < nrows * G; i += kThreads) s_sm[i] = __ldg(S + static_cast<size_t>(n0) * G + i);

    // 2. the next call may start now (its CTAs fit beside this one); the previous one must be done before X is read
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();

    // 3. activations -> three byte planes of 21-bit fixed point, one exponent per 64-element unit.  Thread t
    //    converts elements [16 t, 16 t + 16) (four threads per unit); bytes are stored in the order
    //    k = 8 j + {0,2,4,6 | 1,3,5,7}, the order in which the nibbles of weight word j fall apart into bytes.
    for (int t = tid; t < K / 16; t += kThreads) {
        const uint4* src = reinterpret_cast<const uint4*>(X + 16 * t);
        const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
        const uint32_t u[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        float xf[16];
        float amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            xf[2 * e] = __uint_as_float(u[e] << 16);
            xf[2 * e + 1] = __uint_as_float(u[e] & 0xFFFF0000u);
            amax = max_nan(amax, max_nan(fabsf(xf[2 * e]), fabsf(xf[2 * e + 1])));
        }
        amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        uint32_t eb = (__float_as_uint(amax) >> 23) & 0xFFu;     // biased exponent of the unit's largest magnitude (255: Inf / NaN)
        const bool finite = eb != 255u;
        eb = eb < 40u ? 40u : eb;
        const float scale = __uint_as_float((274u - eb) << 23);    // 2^(20 - (eb - 127)): |x * scale| < 2^21
        int xi[16];
        int sx = 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            // round to nearest integer with the 1.5 * 2^23 trick (no conversion instruction)
            xi[i] = static_cast<int>(__float_as_uint(fmaf(xf[i], scale, 12582912.0f))) - 0x4B400000;
            sx += xi[i];
        }
        sx += __shfl_xor_sync(0xffffffffu, sx, 1);
        sx += __shfl_xor_sync(0xffffffffu, sx, 2);
        if ((t & 3) == 0) {
            inv_sm[t >> 2] = finite ? __uint_as_float((eb - 20u) << 23) : __uint_as_float(0x7FC00000u);   // 1 / scale (NaN for Inf / NaN input)
            sumx_sm[t >> 2] = sx;
        }
        uint32_t pw[3][4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {              // g = 2 * half + parity: elements 8 * half + parity + {0, 2, 4, 6}
            const int base = 8 * (g >> 1) + (g & 1);
            const uint32_t a = xi[base], bb = xi[base + 2], c = xi[base + 4], d = xi[base + 6];
            const uint32_t ab = __byte_perm(a, bb, 0x5140), cd = __byte_perm(c, d, 0x5140);     // [a0 b0 a1 b1], [c0 d0 c1 d1]
            pw[0][g] = __byte_perm(ab, cd, 0x5410);
            pw[1][g] = __byte_perm(ab, cd, 0x7632);
            pw[2][g] = __byte_perm(__byte_perm(a, bb, 0x0062), __byte_perm(c, d, 0x0062), 0x5410);   // signed top bytes
        }
#pragma unroll
        for (int p = 0; p < 3; ++p)
            *reinterpret_cast<uint4*>(planes + static_cast<size_t>(p) * K + static_cast<size_t>(t & 3) * (16 * U) + 16 * (t >> 2)) =
                make_uint4(pw[p][0], pw[p][1], pw[p][2], pw[p][3]);          // [plane][quarter of the unit][unit][16 bytes]
    }
    __syncthreads();                       // planes, scales (when loaded by threads) and the barrier are in shared memory

    // 4. every thread: the planes of its unit into registers, first-read half first
    const int u_idx = tid % U, rs = tid / U;
    const int swap = (lane >> 2) & 1;              // lanes 4-7, 12-15, ... read the upper 16 bytes of their 32 first
    uint32_t P[3][16];
#pragma unroll
    for (int p = 0; p < 3; ++p) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int hh = h ^ swap;               // which half of the unit is read h-th
            // quarters 2 hh and 2 hh + 1 of this unit; consecutive threads read consecutive 16-byte pieces
            const uint4 a = *reinterpret_cast<const uint4*>(planes + static_cast<size_t>(p) * K + static_cast<size_t>(2 * hh) * (16 * U) + 16 * u_idx);
            const uint4 b = *reinterpret_cast<const uint4*>(planes + static_cast<size_t>(p) * K + static_cast<size_t>(2 * hh + 1) * (16 * U) + 16 * u_idx);
            P[p][8 * h + 0] = a.x; P[p][8 * h + 1] = a.y; P[p][8 * h + 2] = a.z; P[p][8 * h + 3] = a.w;
            P[p][8 * h + 4] = b.x; P[p][8 * h + 5] = b.y; P[p][8 * h + 6] = b.z; P[p][8 * h + 7] = b.w;
        }
    }
    const float inv = inv_sm[u_idx];
    const int sumx8 = 8 * sumx_sm[u_idx];

    float acc[kMaxRowsPerThread];
#pragma unroll
    for (int i = 0; i < kMaxRowsPerThread; ++i) acc[i] = 0.0f;
    const bool ok = ptx::mbar_wait(bar, 0, status, 8);          // weights (and scales) have landed
    if (ok) {
#pragma unroll
        for (int i = 0; i < kMaxRowsPerThread; ++i) {
            const int r = rs + RS * i;
            if (r < nrows) {
                const uint8_t* wrow = w_sm + static_cast<size_t>(r) * row_bytes + 32 * u_idx;
                const uint4 wf = *reinterpret_cast<const uint4*>(wrow + 16 * swap);
                const uint4 ws = *reinterpret_cast<const uint4*>(wrow + 16 * (swap ^ 1));
                const float sc = __half2float(s_sm[r * G + (u_idx >> 1)]);
                const uint32_t words[8] = {wf.x, wf.y, wf.z, wf.w, ws.x, ws.y, ws.z, ws.w};
                // six independent chains (three planes x even / odd K): a dp4a waits for the one before it in its chain
                int a0 = 0, a1 = 0, a2 = 0, b0 = 0, b1 = 0, b2 = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // nibbles + 8 as bytes, one logic operation each: even K as q + 8, odd K left in the upper half of
                    // their bytes as 16 (q + 8) — their sums are exact multiples of 16 and lose the factor below
                    const uint32_t ev = (words[j] ^ 0x88888888u) & 0x0F0F0F0Fu;
                    const uint32_t od = (words[j] ^ 0x88888888u) & 0xF0F0F0F0u;
                    a0 = dp4a_uu(ev, P[0][2 * j], a0); b0 = dp4a_uu(od, P[0][2 * j + 1], b0);
                    a1 = dp4a_uu(ev, P[1][2 * j], a1); b1 = dp4a_uu(od, P[1][2 * j + 1], b1);
                    a2 = dp4a_us(ev, P[2][2 * j], a2); b2 = dp4a_us(od, P[2][2 * j + 1], b2);
                }
                a0 += b0 >> 4; a1 += b1 >> 4; a2 += b2 >> 4;       // |b| <= 240 * 255 * 32 < 2^21: no overflow, exact shifts
                // sum over the unit of (q + 8) * x_int, exact in 32 bits (< 2^30); take the 8 * sum(x_int) out again
                // (unsigned arithmetic: the intermediate sums may wrap, the result, |.| <= 2^30, does not)
                const uint32_t tot = (static_cast<uint32_t>(a2) << 16) + (static_cast<uint32_t>(a1) << 8) + static_cast<uint32_t>(a0) -
                                     static_cast<uint32_t>(sumx8);
                acc[i] = static_cast<float>(static_cast<int>(tot)) * (inv * sc);
            }
        }
    }

    // 5. over the U threads of a row.  Inside the warp the (up to) eight row sums of a lane are folded while they are
    //    exchanged (4 + 2 + 1 shuffles leave one row per group of four lanes, two more finish it): lanes 4 s .. 4 s + 3
    //    end up with row slot s; then the row's warps are added in a fixed order.
    {
        float v8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v8[i] = i < kMaxRowsPerThread ? acc[i] : 0.0f;
        float v4[4], v2[2], v1;
        const bool up16 = lane & 16, up8 = lane & 8, up4 = lane & 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float send = up16 ? v8[j] : v8[j + 4];
            const float keep = up16 ? v8[j + 4] : v8[j];
            v4[j] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 16);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float send = up8 ? v4[j] : v4[j + 2];
            const float keep = up8 ? v4[j + 2] : v4[j];
            v2[j] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 8);
        }
        {
            const float send = up4 ? v2[0] : v2[1];
            const float keep = up4 ? v2[1] : v2[0];
            v1 = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 4);
        }
        v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 2);
        v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 1);
        if ((lane & 3) == 0) red[warp * 8 + (lane >> 2)] = v1;
    }
    __syncthreads();
    if (tid < nrows) {
        const int rs_r = tid % RS, i = tid / RS;              // row tid belongs to row set rs_r, pass i
        const int warps_per_rs = U / 32;
        float sum = 0.0f;
        for (int w = 0; w < warps_per_rs; ++w) sum += red[(rs_r * warps_per_rs + w) * 8 + i];
        Y[n0 + tid] = __float2bfloat16_rn(sum);
    }
}

}  // namespace w4s

// Called by b200q_gemm_w4a16 for one token when K is a multiple of 2048 and at most 16384 (K / 64 threads cover a row
// and 256 / (K / 64) rows are in flight per pass).  pdl: launch with programmatic stream serialisation.
int gemm_w4a16_stream(const void* X, const void* Wq, const void* S, void* Y, int N, int K, int group, int pdl, void* stream)
{
    using namespace w4s;
    if (X == nullptr || Wq == nullptr || S == nullptr || Y == nullptr) return cudaErrorInvalidValue;
    if (N <= 0 || K <= 0 || group != kGroup || K % 2048 != 0 || K > 16384) return cudaErrorInvalidValue;
    if (!aligned16(X) || !aligned16(Wq)) return cudaErrorInvalidValue;
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int U = K / kUnit, RS = kThreads / U;
    // Exactly one CTA per SM when a CTA's share then fits (shared memory: kSlabBytes; registers: kMaxRowsPerThread rows
    // per thread), else as many CTAs as that limit asks for.  With programmatic dependent launch, equal grids of one
    // CTA per SM keep the CTAs of consecutive calls spread evenly: a slot freed on an SM is taken by the next call's CTA.
    int max_rows = kSlabBytes / (K / 2);
    if (max_rows > RS * kMaxRowsPerThread) max_rows = RS * kMaxRowsPerThread;
    if (max_rows < 1) return cudaErrorInvalidValue;
    int grid = (N + max_rows - 1) / max_rows;
    if (grid < sms) grid = sms < N ? sms : N;
    const int rows = (N + grid - 1) / grid;                              // the largest share
    uint32_t* status = status_ptr();
    if (status == nullptr) return cudaErrorInvalidDevice;
    const Layout L = layout(K, rows);
    // the scales travel by bulk copy: a row's scales are K / 64 bytes, a multiple of 16 (K % 2048 == 0), so every
    // CTA's piece is aligned when S is
    const int scales_by_copy = aligned16(S) ? 1 : 0;
    constexpr int kMaxSmem = 112 * 1024;
    if (L.total > kMaxSmem) return cudaErrorInvalidValue;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(w4a16_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, w4a16_stream_kernel, static_cast<const __nv_bfloat16*>(X), static_cast<const uint8_t*>(Wq),
                              static_cast<const __half*>(S), static_cast<__nv_bfloat16*>(Y), N, K, rows, scales_by_copy, status);
}

}  // namespace b200q
