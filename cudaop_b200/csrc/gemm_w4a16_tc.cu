// INT4 weight-only decode GEMM on the 5th-generation tensor cores (tcgen05), sm_100a.
//   Y[M,N] (bf16) = X[M,K] (bf16) * dequant(Wq)[N,K]^T,   w[n,k] = q[n,k] * S[n, k/128]
// Wq: two signed nibbles per byte along K, low nibble = lower K
// (op/test/arch_primitives/ptx_mma_integer.cu:93-108); S fp16, one per 128 K, no zero point.
//
// The operation is bound by streaming Wq from HBM once.  The roles are swapped so that nothing is
// wasted on the few tokens: the WEIGHT rows are the M dimension of the MMA (128 rows per CTA) and
// the tokens its N dimension (16).  Per 128-K group:
//   TMA (64-byte swizzle) brings the packed 128 x 64 B weight tile into a shared-memory ring;
//   eight warps (two threads per weight row) turn nibbles into bf16 integers 136 + w in registers
//   (exact: three bit operations per pair, no arithmetic) and store them straight into TENSOR
//   MEMORY (tcgen05.st), so the 4x larger bf16 weights never touch shared memory; the same warps
//   stage the matching 16 x 128 activation tile (bf16, 128-byte swizzle) in shared memory together
//   with the per-token sum of the group's activations (which removes the +136 again, in fp32);
//   one thread issues 8 x tcgen05.mma kind::f16 (128 x 16 x 16), A from TMEM, B from shared memory,
//   into a per-group fp32 accumulator in TMEM;
//   every group has its own accumulator (eight of them), so the warps convert group after group without
//   waiting for a result, and only at the end read the accumulators (tcgen05.ld) and add
//   scale[n, group] * (acc - 136 * sum_x) in fp32 registers: q*s is never rounded.
// Consecutive calls overlap through programmatic dependent launch: a call starts its prologue and
// weight stream while the previous kernel drains, and waits (griddepcontrol.wait) only before it
// touches the activations.
// The MMA contraction index is a dummy, so K inside each 8-element word is permuted
// (0,4,1,5,2,6,3,7: the order in which a 32-bit word yields nibble pairs) identically on both sides.
// K is split over a cluster of CTAs (N/128 row blocks alone would not fill the GPU); the CTAs of a
// cluster add their partial sums through distributed shared memory in a fixed order (deterministic)
// and the leader writes bf16.
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace w4tc {

using ptx::tmem_st_32x32b_x16;
using ptx::tmem_st_wait;
using ptx::tmem_ld_32x32b_x8;
using ptx::umma_f16_ts;
using ptx::pdl_launch_dependents;
using ptx::pdl_wait;
using ptx::ld_dsmem_f32;

constexpr int kRows = 128;          // weight rows per CTA (UMMA M)
constexpr int kTok = 16;            // tokens per pass (UMMA N)
constexpr int kGroup = 128;         // K per scale group
constexpr int kWStages = 8;         // packed weight tiles in flight (8 KiB each)
constexpr int kBatch = 3;            // groups converted per hand-off to the MMA thread (one wait, one fence, one arrive)
constexpr int kASlots = 2 * kBatch;  // TMEM operand slots (64 columns each) with their activation tiles: two batches
constexpr int kDSlots = 8;          // TMEM accumulators (16 columns each): one per group for up to 8 groups per CTA, so
                                    // no worker waits for an MMA result before every group has been converted
constexpr int kWorkers = 256;       // warps 2-9: two threads per weight row (one per 64-K half)
constexpr int kThreads = 64 + kWorkers;   // warp 0 TMA, warp 1 MMA
constexpr int kWTileBytes = kRows * 64;
constexpr int kXTileBytes = 2 * kTok * 128;       // two 64-K sub-tiles of 16 rows x 128 B
constexpr uint32_t kTmemCols = 512;               // 6 x 64 operand columns + 8 x 16 accumulator columns
constexpr int kSmemUsed = kWStages * kWTileBytes + kASlots * kXTileBytes + kRows * kTok * 4 + kDSlots * kTok * 4 + 1024 + 256;
// A CTA takes all 512 TMEM columns, so two CTAs must never share an SM: a second one would block in
// tcgen05.alloc behind the first, and with clusters waiting on their peers that can close a cycle.
// Asking for more than half of the SM's shared memory rules it out.
constexpr int kSmemBytes = kSmemUsed > 120 * 1024 ? kSmemUsed : 120 * 1024;

struct Params {
    const __nv_bfloat16* X;
    const __half* S;
    __nv_bfloat16* Y;
    int M, N, K;
    int groups_total, groups_per_cta;
    uint32_t* status;
};

__global__ void __launch_bounds__(kThreads, 1)
w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmW, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t w_smem = smem_base;                                   // kWStages x 8 KiB, 64-byte swizzle
    const uint32_t x_smem = w_smem + kWStages * kWTileBytes;             // kASlots x 4 KiB, 128-byte swizzle
    const uint32_t red_smem = x_smem + kASlots * kXTileBytes;            // [kTok][kRows] fp32 partial sums
    const uint32_t sx_smem = red_smem + kRows * kTok * 4;                // [kDSlots][kTok] fp32: sum of a group's activations
    const uint32_t bar_base = sx_smem + kDSlots * kTok * 4;
    auto w_full = [&](int s) { return bar_base + 8u * s; };
    auto w_empty = [&](int s) { return bar_base + 8u * (kWStages + s); };
    auto a_ready = [&](int s) { return bar_base + 8u * (2 * kWStages + s); };
    auto a_free = [&](int s) { return bar_base + 8u * (2 * kWStages + 2 + s); };          // a_ready / a_free: per batch parity
    auto d_ready = [&](int s) { return bar_base + 8u * (2 * kWStages + 4 + s); };
    auto d_free = [&](int s) { return bar_base + 8u * (2 * kWStages + 4 + kDSlots + s); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kWStages + 4 + 2 * kDSlots);
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kpart = ptx::cluster_ctarank();              // K slice of this CTA inside its cluster
    const int nsplit = gridDim.x;
    const int n0 = blockIdx.y * kRows;
    const int m0 = blockIdx.z * kTok;
    const int g_begin = kpart * p.groups_per_cta;
    const int g_end = min(g_begin + p.groups_per_cta, p.groups_total);
    const int ngroups = max(g_end - g_begin, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWStages; ++s) { ptx::mbar_init(w_full(s), 1); ptx::mbar_init(w_empty(s), 8); }
        for (int s = 0; s < 2; ++s) { ptx::mbar_init(a_ready(s), 8); ptx::mbar_init(a_free(s), 1); }
        for (int s = 0; s < kDSlots; ++s) { ptx::mbar_init(d_ready(s), 1); ptx::mbar_init(d_free(s), 8); }
        ptx::fence_mbar_init();
    }
    if (warp == 1) { ptx::tmem_alloc(tmem_slot, kTmemCols); ptx::tmem_relinquish(); }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    pdl_launch_dependents();        // the next call may begin: its weights do not depend on this call
    const uint32_t tmem_base = *tmem_slot_ptr;
    const uint32_t a_tmem0 = tmem_base;                       // kASlots x 64 columns: bf16 weights, 2 per column
    const uint32_t d_tmem0 = tmem_base + kASlots * 64;        // kDSlots x 16 columns: fp32 group accumulators

    if (warp == 0) {
        // ------------------------------------------------ TMA: packed weight tiles, independent of X
        if (ptx::elect_one()) {
            ptx::tma_prefetch_desc(&tmW);
            bool ok = true;
            for (int i = 0; i < ngroups && ok; ++i) {
                const int s = i % kWStages;
                if (!ptx::mbar_wait(w_empty(s), ((i / kWStages) & 1u) ^ 1u, p.status, 21)) { ok = false; break; }
                ptx::mbar_arrive_expect_tx(w_full(s), kWTileBytes);
                ptx::tma_load_2d(w_smem + s * kWTileBytes, &tmW, w_full(s), (g_begin + i) * 64, n0);
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            // bf16 x bf16 -> fp32, both K-major, M = 128 weight rows, N = 16 tokens
            constexpr uint32_t idesc = ptx::umma_idesc(1, 1, kRows, kTok);
            bool ok = true;
            for (int b = 0; b * kBatch < ngroups && ok; ++b) {
                const int S = b & 1;
                if (!ptx::mbar_wait(a_ready(S), (b >> 1) & 1u, p.status, 22)) { ok = false; break; }
                for (int gi = 0; gi < kBatch && ok; ++gi) {
                    const int i = b * kBatch + gi;
                    if (i >= ngroups) break;
                    const int s = i % kASlots, ds = i % kDSlots;
                    if (!ptx::mbar_wait(d_free(ds), ((i / kDSlots) & 1u) ^ 1u, p.status, 23)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t xs = x_smem + s * kXTileBytes;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {       // 16 K per instruction: 8 TMEM columns of A, 32 bytes of B
                        const uint64_t db = ptx::smem_desc_sw128_kmajor(xs + (j >> 2) * (kTok * 128)) + 2u * (j & 3);
                        umma_f16_ts(d_tmem0 + ds * kTok, a_tmem0 + s * 64 + j * 8, db, idesc, j != 0);
                    }
                    ptx::umma_commit(d_ready(ds));
                }
                if (ok) ptx::umma_commit(a_free(S));
            }
            if (!ok) __nanosleep(200000);
        }
    } else {
        // ------------------------------------------------ workers: dequant + scale-accumulate.
        // Thread (row, half): row = TMEM lane = weight row in the tile; half = which 64 K of every
        // group it converts and which 8 tokens of the accumulator it folds in.
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row = q * 32 + lane;
        const int n = n0 + row;
        const int tid = threadIdx.x - 64;                      // 0..255 for activation staging
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        float acc[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) acc[m] = 0.0f;
        bool ok = true;
        float* sx = reinterpret_cast<float*>(smem_gen + (sx_smem - smem_base));

        // activation chunk of this thread for a group: token xm, 16-byte chunk xq (of 16 per row)
        const int xm = tid >> 4, xq = tid & 15;
        const bool xvalid = (m0 + xm) < p.M;
        auto load_x = [&](int g) {
            const uint4* src = reinterpret_cast<const uint4*>(p.X + static_cast<size_t>(m0 + xm) * p.K + static_cast<size_t>(g) * kGroup);
            return xvalid ? __ldg(src + xq) : make_uint4(0, 0, 0, 0);
        };
        auto load_scale = [&](int g) {
            return (n < p.N) ? __half2float(__ldg(p.S + static_cast<size_t>(n) * p.groups_total + g)) : 0.0f;
        };
        // the scales of this CTA's first groups (weights: independent of the previous kernel), all requested now so
        // that their latencies overlap; the usual case has at most kDSlots groups per CTA and needs no others
        float scs[kDSlots];
#pragma unroll
        for (int j = 0; j < kDSlots; ++j) scs[j] = (j < ngroups) ? load_scale(g_begin + j) : 0.0f;
        pdl_wait();                                            // the activations may come from the previous kernel
        uint4 xr[kBatch];
#pragma unroll
        for (int gi = 0; gi < kBatch; ++gi) xr[gi] = (gi < ngroups) ? load_x(g_begin + gi) : make_uint4(0, 0, 0, 0);

        // accumulator of group i (finished long ago when this is called): sum_k w x = sum_k (136 + w) x - 136 * sum_k x,
        // times the group's scale, into this thread's fp32 sums
        auto fold = [&](int i, float sc) -> bool {
            const int ds = i % kDSlots;
            if (!ptx::mbar_wait(d_ready(ds), (i / kDSlots) & 1u, p.status, 26)) return false;
            ptx::tcgen05_fence_after_sync();
            uint32_t d[8];
            tmem_ld_32x32b_x8(d_tmem0 + lane_addr + ds * kTok + half * 8, d);
            ptx::tmem_ld_wait();
            float sxv[8];
#pragma unroll
            for (int m = 0; m < 8; ++m) sxv[m] = sx[ds * kTok + half * 8 + m];
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(d_free(ds));
#pragma unroll
            for (int m = 0; m < 8; ++m) acc[m] = fmaf(fmaf(-136.0f, sxv[m], __uint_as_float(d[m])), sc, acc[m]);
            return true;
        };

        // Groups go to the MMA thread in batches of kBatch: one tcgen05.wait::st, one pair of fences and one
        // barrier arrival per batch — the hand-off, not the conversion, is what a group costs.
        for (int b = 0; b * kBatch < ngroups && ok; ++b) {
            const int S = b & 1;
            // more than kDSlots groups per CTA: an accumulator (and its sx row) is reused, fold the old one in first
#pragma unroll
            for (int gi = 0; gi < kBatch; ++gi) {
                const int i = b * kBatch + gi;
                if (ok && i < ngroups && i >= kDSlots) {
                    if (!fold(i - kDSlots, load_scale(g_begin + i - kDSlots))) ok = false;
                    else if (!ptx::mbar_wait(d_free(i % kDSlots), ((i / kDSlots) & 1u) ^ 1u, p.status, 28)) ok = false;   // every worker has read that sx row
                }
            }
            if (!ok) break;
            // the operand slots of this batch parity (TMEM columns + activation tiles) are free once the MMAs of batch b - 2 retired
            if (!ptx::mbar_wait(a_free(S), ((b >> 1) & 1u) ^ 1u, p.status, 24)) { ok = false; break; }
            ptx::tcgen05_fence_after_sync();
#pragma unroll
            for (int gi = 0; gi < kBatch; ++gi) {
                const int i = b * kBatch + gi;
                if (i < ngroups) {
                    // stage the group's activations: K-permuted inside every 8 (x0,x4,x1,x5,x2,x6,x3,x7), 128-byte swizzle;
                    // and the sum of the group's activations per token (for the +136 offset of the weights)
                    uint8_t* xt = smem_gen + (x_smem - smem_base) + (i % kASlots) * kXTileBytes;
                    const int h = xq >> 3, xc = xq & 7;
                    const uint32_t off = h * (kTok * 128) + (xm >> 3) * 1024 + (xm & 7) * 128 + ((xc ^ (xm & 7)) << 4);
                    const uint4 x4 = xr[gi];
                    *reinterpret_cast<uint4*>(xt + off) =
                        make_uint4(__byte_perm(x4.x, x4.z, 0x5410), __byte_perm(x4.x, x4.z, 0x7632),
                                   __byte_perm(x4.y, x4.w, 0x5410), __byte_perm(x4.y, x4.w, 0x7632));
                    const uint32_t w[4] = {x4.x, x4.y, x4.z, x4.w};
                    float t = 0.0f;
#pragma unroll
                    for (int k = 0; k < 4; ++k) t += __uint_as_float(w[k] << 16) + __uint_as_float(w[k] & 0xFFFF0000u);
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);   // the 16 chunks of a token sit in 16 adjacent lanes
                    if (xq == 0) sx[(i % kDSlots) * kTok + xm] = t;
                }
            }
#pragma unroll
            for (int gi = 0; gi < kBatch; ++gi) {              // prefetch the next batch's activations
                const int i = (b + 1) * kBatch + gi;
                if (i < ngroups) xr[gi] = load_x(g_begin + i);
            }
#pragma unroll
            for (int gi = 0; gi < kBatch; ++gi) {
                const int i = b * kBatch + gi;
                if (ok && i < ngroups) {
                    const int ws = i % kWStages, s = i % kASlots;
                    // packed weights of this row: this thread converts 32 of its 64 bytes (64-byte-swizzled by TMA)
                    if (!ptx::mbar_wait(w_full(ws), (i / kWStages) & 1u, p.status, 25)) { ok = false; }
                    else {
                        const uint8_t* wt = smem_gen + (w_smem - smem_base) + ws * kWTileBytes + row * 64;
                        const int sw = (row >> 1) & 3;
#pragma unroll
                        for (int cc = 0; cc < 2; ++cc) {                   // 16 bytes = 32 weights = 16 TMEM columns
                            const int c = 2 * half + cc;
                            const uint4 w4 = *reinterpret_cast<const uint4*>(wt + ((c ^ sw) << 4));
                            const uint32_t ww[4] = {w4.x ^ 0x88888888u, w4.y ^ 0x88888888u, w4.z ^ 0x88888888u, w4.w ^ 0x88888888u};
                            uint32_t r[16];
#pragma unroll
                            for (int k = 0; k < 4; ++k) {                  // nibble pairs (i, i+4) -> bf16 (136 + w): exact integers
                                r[4 * k + 0] = (ww[k] & 0x000F000Fu) | 0x43004300u;
                                r[4 * k + 1] = ((ww[k] >> 4) & 0x000F000Fu) | 0x43004300u;
                                r[4 * k + 2] = ((ww[k] >> 8) & 0x000F000Fu) | 0x43004300u;
                                r[4 * k + 3] = ((ww[k] >> 12) & 0x000F000Fu) | 0x43004300u;
                            }
                            tmem_st_32x32b_x16(a_tmem0 + lane_addr + s * 64 + c * 16, r);
                        }
                    }
                }
            }
            if (!ok) break;
            tmem_st_wait();
            ptx::fence_proxy_async_smem();                     // the activation tiles were written by ordinary stores
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(a_ready(S));
                for (int gi = 0; gi < kBatch; ++gi)
                    if (b * kBatch + gi < ngroups) ptx::mbar_arrive(w_empty((b * kBatch + gi) % kWStages));
            }
        }
        // the accumulators still in tensor memory (all of them when the CTA has at most kDSlots groups)
        if (ngroups <= kDSlots) {
#pragma unroll
            for (int j = 0; j < kDSlots; ++j)
                if (ok && j < ngroups && !fold(j, scs[j])) ok = false;
        } else {
            for (int i = ngroups - kDSlots; i < ngroups && ok; ++i)
                if (!fold(i, load_scale(g_begin + i))) ok = false;
        }
        // partial sums of this K slice: [token][row] so that the cluster reduction reads rows contiguously
        float* red = reinterpret_cast<float*>(smem_gen + (red_smem - smem_base));
#pragma unroll
        for (int m = 0; m < 8; ++m) red[(half * 8 + m) * kRows + row] = acc[m];
    }

    // ---- cluster reduction over the K slices (fixed order), leader writes the output
    ptx::tcgen05_fence_before_sync();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (kpart == 0 && warp >= 2) {
        const int row = (warp & 3) * 32 + lane, half = (warp - 2) >> 2;
        const int n = n0 + row;
        float v[8][8];                                // [peer][token]: all loads issued before any addition
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const uint32_t peer = ptx::mapa(red_smem, r < nsplit ? r : 0);
#pragma unroll
            for (int m = 0; m < 8; ++m)
                v[r][m] = (r < nsplit) ? ld_dsmem_f32(peer + ((half * 8 + m) * kRows + row) * 4) : 0.0f;
        }
        float tot[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) tot[m] = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r)                   // fixed order over the K slices
#pragma unroll
            for (int m = 0; m < 8; ++m) tot[m] += v[r][m];
        if (n < p.N)
#pragma unroll
            for (int m = 0; m < 8; ++m)
                if (m0 + half * 8 + m < p.M) p.Y[static_cast<size_t>(m0 + half * 8 + m) * p.N + n] = __float2bfloat16_rn(tot[m]);
    }
    ptx::cluster_arrive();          // peers keep their shared memory alive until the leader has read it
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

int g_impl = 0;      // 0 = by M: streaming GEMV (gemm_w4a16_stream.cu; the older GEMV forms of gemm_w4a16_gemv.cu when K does not suit it)
                     // for one token, the prefill kernel with the weights in tensor memory (gemm_w4a16_prefill_ts.cu) from 64
                     // tokens on (from 17 when N >= 8192), else the warp-MMA kernel (gemm_w4a16.cu); 5 = the streaming GEMV where it applies; 8 = that prefill
                     // kernel for every M; 6 / 7 = the prefill kernel that converts through shared memory (gemm_w4a16_prefill.cu;
                     // offset taken out by rows of ones / by the converters);
                     // 1 = tcgen05 kernel (this file); 2 = warp-MMA kernel for every M; 3 / 4 = GEMV up to 4 tokens, weights
                     // through shared memory (dp4a arithmetic) / in registers (fp32 arithmetic)
int g_pdl = 0;       // programmatic dependent launch (b200q_w4a16_set_pdl) of the GEMV and tcgen05 kernels, off by default

}  // namespace w4tc
}  // namespace b200q

extern "C" int b200q_gemm_w4a16_warp_mma(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K,
                                         int group, void* stream);
namespace b200q {

// gemm_w4a16_gemv.cu: CUDA-core kernel for M <= 4
int gemm_w4a16_gemv(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int group, int pdl, int form,
                    void* stream);
// gemm_w4a16_stream.cu: one token, fat CTAs that prefetch their whole weight block (K % 2048 == 0, K <= 16384)
int gemm_w4a16_stream(const void* X, const void* Wq, const void* S, void* Y, int N, int K, int group, int pdl, void* stream);
// gemm_w4a16_prefill.cu: many tokens, tcgen05 with group-wise partial-sum scaling (K % 128 == 0, K <= 16384)
int gemm_w4a16_prefill(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int group, int sub, void* stream);
// gemm_w4a16_prefill_ts.cu: many tokens, the converted weights as the tensor-memory operand (K % 128 == 0)
int gemm_w4a16_prefill_ts(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int group, void* stream);
}

extern "C" int b200q_w4a16_set_impl(int impl)
{
    if (impl < 0 || impl > 8) return cudaErrorInvalidValue;
    b200q::w4tc::g_impl = impl;
    return 0;
}

extern "C" int b200q_w4a16_set_pdl(int on)
{
    b200q::w4tc::g_pdl = on ? 1 : 0;
    return 0;
}

extern "C" int b200q_gemm_w4a16(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int group,
                                void* stream)
{
    using namespace b200q;
    // measured crossover against the warp-MMA kernel: from 64 tokens on, and from 17 where the weight rows alone
    // fill the machine's tiles (N >= 8192)
    if (((M > 16 && (M >= 64 || N >= 8192) && w4tc::g_impl == 0) || w4tc::g_impl == 8) && group == 128 && K > 0 && K % 128 == 0)
        return gemm_w4a16_prefill_ts(X, Wq, S, Y, M, N, K, group, stream);
    if ((w4tc::g_impl == 6 || w4tc::g_impl == 7) && group == 128 && K > 0 && K % 128 == 0 && K <= 16384)
        return gemm_w4a16_prefill(X, Wq, S, Y, M, N, K, group, w4tc::g_impl == 7 ? 1 : 0, stream);
    if (M == 1 && (w4tc::g_impl == 0 || w4tc::g_impl == 5) && group == 128 && K > 0 && K % 2048 == 0 && K <= 16384)
        return gemm_w4a16_stream(X, Wq, S, Y, N, K, group, w4tc::g_pdl, stream);
    if (M == 1 && (w4tc::g_impl == 0 || w4tc::g_impl == 5)) {
        // one token: CUDA cores.  Measured (K = 4096, 80 weight sets cycled in a graph): up to 8 MiB of weights the
        // form with the weights in registers is ahead (4096 rows: 4.7 vs 5.1 us), beyond it the shared-memory /
        // dp4a form (8192 rows: 6.6 vs 8.4 us).
        const bool big = static_cast<long long>(N) * (K / 2) > (8ll << 20);
        return gemm_w4a16_gemv(X, Wq, S, Y, M, N, K, group, w4tc::g_pdl, big ? 0 : 1, stream);
    }
    if (M <= 4 && (w4tc::g_impl == 3 || w4tc::g_impl == 4))
        return gemm_w4a16_gemv(X, Wq, S, Y, M, N, K, group, w4tc::g_pdl, w4tc::g_impl == 4 ? 1 : 0, stream);
    if (w4tc::g_impl != 1) return b200q_gemm_w4a16_warp_mma(X, Wq, S, Y, M, N, K, group, stream);
    if (X == nullptr || Wq == nullptr || S == nullptr || Y == nullptr) return cudaErrorInvalidValue;
    if (M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
    if (group != w4tc::kGroup || K % w4tc::kGroup != 0) return cudaErrorInvalidValue;
    if (!aligned16(X) || !aligned16(Wq)) return cudaErrorInvalidValue;

    w4tc::Params p{};
    p.X = static_cast<const __nv_bfloat16*>(X); p.S = static_cast<const __half*>(S); p.Y = static_cast<__nv_bfloat16*>(Y);
    p.M = M; p.N = N; p.K = K; p.groups_total = K / w4tc::kGroup;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int row_blocks = (N + w4tc::kRows - 1) / w4tc::kRows;
    int split = 1;                                        // K slices = cluster size: fill the SMs, keep >= 1 group each
    while (split < 8 && row_blocks * split * 2 <= sms + sms / 4 && split * 2 <= p.groups_total) split *= 2;
    p.groups_per_cta = (p.groups_total + split - 1) / split;

    CUtensorMap tmW;
    if (!make_tmap_2d_u8(&tmW, Wq, N, K / 2, K / 2, w4tc::kRows, 64, CU_TENSOR_MAP_SWIZZLE_64B)) return cudaErrorInvalidValue;

    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(w4tc::w4a16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, w4tc::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(split, row_blocks, (M + w4tc::kTok - 1) / w4tc::kTok);
    cfg.blockDim = dim3(w4tc::kThreads);
    cfg.dynamicSmemBytes = w4tc::kSmemBytes;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: this call may start while the previous kernel of the stream drains
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = w4tc::g_pdl ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, w4tc::w4a16_tc_kernel, tmW, p);
}
