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

using ptx::max_nan;
using ptx::dp4a_uu;
using ptx::dp4a_us;
using ptx::bulk_load;

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
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();

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


// ------------------------------------------------------------------------------------------------------
// Second form (larger matrices): the CTA's whole share of Wq lands in shared memory with ONE bulk copy (its
// rows are contiguous in memory), so nothing but an mbarrier is held while the data is in flight: under 64
// registers per thread and 15 KiB of shared memory per CTA, four CTAs per SM — small enough that the CTAs
// of the NEXT call (programmatic dependent launch) become resident and stream their weights while this
// call computes.  Warp = K slice, as above; it walks the CTA's rows (at most kMaxRows), reading its 16
// bytes per row from shared memory.  The arithmetic is integer: a lane turns its 32 activations once into
// 21-bit fixed point relative to the chunk's largest exponent (every bf16 within 2^13 of the largest is
// exact, the rest is off by at most 2^-22 of it — below the fp32 accumulation noise of the reference),
// split into three byte planes; a weight word falls apart into two words of four nibble-bytes (q + 8) with
// three logic operations, and six dp4a per word accumulate the exact 32-bit sum of (q + 8) * x_int.
// 8 * sum(x_int) is subtracted, the result converted once per row and chunk and scaled by 2^-shift * S in
// fp32.  About 1.1 instructions per weight instead of 3.
constexpr int kMaxRows = 8;


template <int MT>
__global__ void __launch_bounds__(256)
w4a16_gemv_smem_kernel(const __nv_bfloat16* __restrict__ X, const uint8_t* __restrict__ Wq, const __half* __restrict__ S,
                       __nv_bfloat16* __restrict__ Y, int M, int N, int K, int rows_per_cta, uint32_t* status)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x, ks = threadIdx.y;
    const int slices = blockDim.y;
    const int tid = ks * 32 + lane, nthreads = slices * 32;
    const int G = K / kGroup;
    const int n0 = blockIdx.x * rows_per_cta;
    const int nrows = min(rows_per_cta, N - n0);
    const int m0 = blockIdx.y * MT;
    const uint32_t w_bytes = static_cast<uint32_t>(nrows) * (K / 2);
    uint8_t* w_sm = smem;                                                        // [nrows][K/2]
    __half* s_sm = reinterpret_cast<__half*>(smem + static_cast<size_t>(rows_per_cta) * (K / 2));   // [nrows][G]
    float* red = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s_sm) + ((rows_per_cta * G * 2 + 15) & ~15));  // [slices][kMaxRows*MT]
    const uint32_t bar = ptx::smem_u32(red + slices * kMaxRows * MT);

    // 1. the weights of this CTA: one bulk copy; the scales: a few plain loads.  Neither depends on the
    //    kernel before this one.
    if (tid == 0) {
        ptx::mbar_init(bar, 1);
        ptx::fence_mbar_init();
        ptx::mbar_arrive_expect_tx(bar, w_bytes);
        bulk_load(ptx::smem_u32(w_sm), Wq + static_cast<size_t>(n0) * (K / 2), w_bytes, bar);
    }
    for (int i = tid; i < nrows * G; i += nthreads) s_sm[i] = __ldg(S + static_cast<size_t>(n0) * G + i);

    // 2. the next call may start now (its CTAs fit beside these); wait for the previous one before X
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();

    float acc[kMaxRows][MT];
#pragma unroll
    for (int r = 0; r < kMaxRows; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

    __syncthreads();                 // barrier initialised, scales in shared memory
    bool ok = true;
    for (int k0 = ks * kSliceK + lane * 32; k0 < K; k0 += slices * kSliceK) {
        // Activations of this lane's 32 K as 21-bit fixed point relative to the chunk's largest exponent
        // (exact for every bf16 within 2^13 of the largest, 2^-22 of it otherwise), split into three byte
        // planes laid out the way the nibbles of a weight word fall apart into bytes:
        // plane[p][2q] holds k = 8q + {0,2,4,6}, plane[p][2q+1] holds k = 8q + {1,3,5,7}.
        uint32_t plane[MT][3][8];
        int sumx[MT];
        float inv[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const bool in = (m0 + m) < M;
            const uint4* src = reinterpret_cast<const uint4*>(X + static_cast<size_t>(in ? m0 + m : 0) * K + k0);
            float xf[32];
            float amax = 0.0f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 v = in ? __ldg(src + q) : make_uint4(0, 0, 0, 0);
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    xf[8 * q + 2 * e] = __uint_as_float(u[e] << 16);
                    xf[8 * q + 2 * e + 1] = __uint_as_float(u[e] & 0xFFFF0000u);
                    amax = max_nan(amax, max_nan(fabsf(xf[8 * q + 2 * e]), fabsf(xf[8 * q + 2 * e + 1])));
                }
            }
            uint32_t eb = (__float_as_uint(amax) >> 23) & 0xFFu;     // biased exponent of the largest magnitude (255: Inf or NaN)
            const bool finite = eb != 255u;
            eb = eb < 40u ? 40u : eb;
            const float scale = __uint_as_float((274u - eb) << 23);    // 2^(20 - (eb - 127)): |x * scale| < 2^21
            inv[m] = finite ? __uint_as_float((eb - 20u) << 23) : __uint_as_float(0x7FC00000u);   // 1 / scale (NaN for Inf/NaN input)
            int xi[32];
            int sx = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                // round to nearest integer with the 1.5 * 2^23 trick (no conversion instruction)
                xi[i] = static_cast<int>(__float_as_uint(fmaf(xf[i], scale, 12582912.0f))) - 0x4B400000;
                sx += xi[i];
            }
            sumx[m] = sx;
#pragma unroll
            for (int g = 0; g < 8; ++g) {          // g = 2q + parity: values k = 8q + parity + {0, 2, 4, 6}
                const int base = 8 * (g >> 1) + (g & 1);
                const uint32_t a = xi[base], bb = xi[base + 2], c = xi[base + 4], d = xi[base + 6];
                const uint32_t ab = __byte_perm(a, bb, 0x5140), cd = __byte_perm(c, d, 0x5140);     // [a0 b0 a1 b1], [c0 d0 c1 d1]
                plane[m][0][g] = __byte_perm(ab, cd, 0x5410);
                plane[m][1][g] = __byte_perm(ab, cd, 0x7632);
                plane[m][2][g] = __byte_perm(__byte_perm(a, bb, 0x0062), __byte_perm(c, d, 0x0062), 0x5410);   // signed top bytes
            }
        }
        if (ok && !ptx::mbar_wait(bar, 0, status, 7)) ok = false;          // weights have landed (only the first pass waits)
        if (!ok) break;
#pragma unroll
        for (int r = 0; r < kMaxRows; ++r) {
            if (r < nrows) {
                const uint4 w = *reinterpret_cast<const uint4*>(w_sm + static_cast<size_t>(r) * (K / 2) + k0 / 2);
                const float sc = __half2float(s_sm[r * G + k0 / kGroup]);
                const uint32_t words[4] = {w.x, w.y, w.z, w.w};
                int a0[MT], a1[MT], a2[MT];
#pragma unroll
                for (int m = 0; m < MT; ++m) { a0[m] = 0; a1[m] = 0; a2[m] = 0; }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    // nibbles + 8 as bytes: even K in one word, odd K in the other
                    const uint32_t ev = (words[q] ^ 0x88888888u) & 0x0F0F0F0Fu;
                    const uint32_t od = ((words[q] >> 4) ^ 0x08080808u) & 0x0F0F0F0Fu;
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        a0[m] = dp4a_uu(ev, plane[m][0][2 * q], a0[m]);
                        a0[m] = dp4a_uu(od, plane[m][0][2 * q + 1], a0[m]);
                        a1[m] = dp4a_uu(ev, plane[m][1][2 * q], a1[m]);
                        a1[m] = dp4a_uu(od, plane[m][1][2 * q + 1], a1[m]);
                        a2[m] = dp4a_us(ev, plane[m][2][2 * q], a2[m]);
                        a2[m] = dp4a_us(od, plane[m][2][2 * q + 1], a2[m]);
                    }
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    // sum over the chunk of (q + 8) * x_int, exact in 32 bits; take the 8 * sum(x_int) out again
                    const int tot = (a2[m] << 16) + (a1[m] << 8) + a0[m] - 8 * sumx[m];
                    acc[r][m] = fmaf(static_cast<float>(tot) * inv[m], sc, acc[r][m]);
                }
            }
        }
    }

    // over the lanes, then over the K slices in a fixed order
#pragma unroll
    for (int r = 0; r < kMaxRows; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[r][m];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
            if (lane == 0) red[ks * (kMaxRows * MT) + r * MT + m] = v;
        }
    __syncthreads();
    if (tid < kMaxRows * MT) {
        const int r = tid / MT, m = tid % MT;
        float sum = 0.0f;
        for (int j = 0; j < slices; ++j) sum += red[j * (kMaxRows * MT) + tid];
        if (r < nrows && m0 + m < M) Y[static_cast<size_t>(m0 + m) * N + n0 + r] = __float2bfloat16_rn(sum);
    }
}

}  // namespace w4gemv

// Called by b200q_gemm_w4a16 for M <= 4.  pdl: launch with programmatic stream serialisation, i.e. this
// kernel may start (and stream its weights) while the previous kernel of the stream is still running.
// form 0: weights through shared memory (bulk copy), 1: weights in registers.
int gemm_w4a16_gemv(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int group, int pdl, int form,
                    void* stream)
{
    using namespace w4gemv;
    if (X == nullptr || Wq == nullptr || S == nullptr || Y == nullptr) return cudaErrorInvalidValue;
    if (M <= 0 || M > 4 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
    if (group != kGroup || K % kGroup != 0) return cudaErrorInvalidValue;
    if (!aligned16(X) || !aligned16(Wq)) return cudaErrorInvalidValue;
    const int all_slices = (K + kSliceK - 1) / kSliceK;
    const int slices = all_slices < kMaxSliceWarps ? all_slices : kMaxSliceWarps;     // warps per row block
    const int mt = (M == 1) ? 1 : 2;
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(X);
    const uint8_t* wq = static_cast<const uint8_t*>(Wq);
    const __half* s = static_cast<const __half*>(S);
    __nv_bfloat16* y = static_cast<__nv_bfloat16*>(Y);
    cudaLaunchConfig_t cfg{};
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;

    if (form == 0 && K / 2 <= 48 * 1024) {
        const int sms = num_sms();
        if (sms <= 0) return cudaErrorInvalidDevice;
        int rows = 48 * 1024 / (K / 2);                       // what fits in 48 KiB of shared memory
        if (rows > kMaxRows) rows = kMaxRows;
        const int want = (N + 4 * sms - 1) / (4 * sms);      // four CTAs per SM
        if (rows > want) rows = want;
        uint32_t* status = status_ptr();
        if (status == nullptr) return cudaErrorInvalidDevice;
        const int G = K / kGroup;
        cfg.gridDim = dim3((N + rows - 1) / rows, (M + mt - 1) / mt);
        cfg.blockDim = dim3(32, slices, 1);
        cfg.dynamicSmemBytes = static_cast<size_t>(rows) * (K / 2) + ((rows * G * 2 + 15) & ~15) +
                               static_cast<size_t>(slices) * kMaxRows * mt * sizeof(float) + 16;
        static bool configured[64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 64 && !configured[dev]) {
            e = cudaFuncSetAttribute(w4a16_gemv_smem_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(w4a16_gemv_smem_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
            if (e != cudaSuccess) return e;
            configured[dev] = true;
        }
        if (mt == 1) return cudaLaunchKernelEx(&cfg, w4a16_gemv_smem_kernel<1>, x, wq, s, y, M, N, K, rows, status);
        return cudaLaunchKernelEx(&cfg, w4a16_gemv_smem_kernel<2>, x, wq, s, y, M, N, K, rows, status);
    }

    const int rbs = slices >= 4 ? 1 : 4 / slices;              // at least four warps per CTA
    cfg.gridDim = dim3((N + rbs * kRows - 1) / (rbs * kRows), (M + mt - 1) / mt);
    cfg.blockDim = dim3(32, slices, rbs);
    cfg.dynamicSmemBytes = static_cast<size_t>(rbs) * slices * kRows * mt * sizeof(float);
    if (mt == 1) return cudaLaunchKernelEx(&cfg, w4a16_gemv_kernel<1>, x, wq, s, y, M, N, K);
    return cudaLaunchKernelEx(&cfg, w4a16_gemv_kernel<2>, x, wq, s, y, M, N, K);
}

}  // namespace b200q
