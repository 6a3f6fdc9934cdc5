// INT4 weight-only GEMM for prefill shapes (many tokens) on the 5th-generation tensor cores, sm_100a.
//   Y[M,N] (bf16) = X[M,K] (bf16) * dequant(Wq)[N,K]^T,   w[n,k] = q[n,k] * S[n, k/128]
// Wq: two signed nibbles per byte along K, low nibble = lower K
// (op/test/arch_primitives/ptx_mma_integer.cu:93-108); S fp16, one per 128 K, no zero point.
//
// With hundreds of tokens the operation is compute-bound, and the per-group scales are what shapes the kernel:
// q * s must not be rounded to bf16 (that alone costs about 1e-3 relative error), so the tensor core multiplies
// the activations by the INTEGER weights, one 128-K group at a time, and the group's scale is applied to the fp32
// partial sum afterwards — "group-wise partial-sum scaling".
//   tile      128 tokens x 128 weight rows per CTA, persistent over tiles; consecutive tiles share the token rows
//   warp 0    TMA producer: per 64 K the 128 x 64 activation tile (128-byte swizzle) and the packed 128 x 32-byte
//             weight tile into a four-stage ring (two stages per scale group)
//   warps 10-13 converters (one thread per weight row): nibble pairs -> bf16 integers 136 + q with one logic operation per pair (exact, no
//             arithmetic), re-paired into ascending K order with one byte permute per pair and written as the
//             128-byte-swizzled K-major B tile the MMA reads.  Sixteen more B rows hold the constant 1.0, so the
//             tensor core also delivers sum_k x per token and group, which takes the offset 136 out again.
//   warp 1    MMA issuer: 4 x tcgen05.mma kind::f16 (128 x 144 x 16) per stage, a group into one of two TMEM accumulators
//   warps 2-9 fold: tcgen05.ld the group's accumulator (two warps per lane quadrant, 64 weight rows each) and add
//             scale[n, g] * (acc[n] - 136 * acc[ones]) into fp32 registers; after the last group: bf16, 16-byte stores.
// fp32 accumulation inside a group (tensor core) and across groups (registers); one rounding at the end.
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace w4p {

constexpr int kBM = 128;             // tokens per tile (UMMA M)
constexpr int kBN = 128;             // weight rows per tile
constexpr int kBNmma = kBN + 16;     // + sixteen rows of ones (UMMA N, a multiple of 16)
constexpr int kGroup = 128;          // K per scale group
constexpr int kBK = 64;              // K per pipeline stage: one 128-byte swizzle row of bf16; two stages per group
constexpr int kMaxLoadStages = 12;   // ring of TMA destinations (activations + packed weights); its depth is set per launch
constexpr int kMaxWbStages = 4;      // ring of converted weight tiles
constexpr int kMaxGroups = 128;      // scales of a tile are staged in shared memory: K <= 16384
constexpr int kXBytes = kBM * 128;                 // 16 KiB
constexpr int kWpBytes = kBN * 32;                 // packed weights of a stage, 4 KiB
constexpr int kWbBytes = kBNmma * 128;             // converted weights, 18 KiB
constexpr int kLoadBytes = kXBytes + kWpBytes;     // 20 KiB per load stage

constexpr int kFoldWarps = 8, kConvWarps = 4;     // converter warps per team; one team converts a stage
constexpr int kThreads = 32 * (2 + kFoldWarps + kConvWarps);
constexpr uint32_t kTmemCols = 512;                // two accumulators of 144 columns (allocations are powers of two)
constexpr int kAccStride = 160;                    // columns between the two accumulators
constexpr int kBarBytes = 512;
constexpr int kMaxSmemBytes = 232448;              // 227 KiB per CTA
static_assert(kXBytes % 1024 == 0 && kWpBytes % 1024 == 0 && kWbBytes % 1024 == 0, "operand tiles start 1024-byte aligned");

// (136 + q, 136 + q') as bf16x2 -> (q, q'): exact, both sides are integers below 256
__device__ __forceinline__ uint32_t sub136(uint32_t v)
{
    const uint32_t k = 0x43084308u;
    const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v), *reinterpret_cast<const __nv_bfloat162*>(&k));
    return *reinterpret_cast<const uint32_t*>(&r);
}

struct Params {
    const __half* S;
    __nv_bfloat16* Y;
    int M, N, K;
    int tiles_m, tiles_n;
    int load_stages;      // depth of the TMA ring: as deep as shared memory allows beside the scales of K / 128 groups
    uint32_t* status;
};

// SUB: the converters subtract the offset again (one exact bf16x2 subtraction per pair: 136 + q and q are both
// bf16 integers), the B tile holds q itself, no rows of ones are multiplied and the fold is one fused
// multiply-add per value.
// Two teams of four converter warps: team t converts the stages whose running index is t modulo 2 (measured: +12 %
// over one team; wider tcgen05.ld in the fold and a deeper load ring changed nothing).
constexpr int kTeams = 2;
template <bool SUB>
__global__ void __launch_bounds__(kThreads + 32 * kConvWarps * (kTeams - 1), 1)
w4a16_prefill_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    constexpr int kWS = 4;                  // converted tiles in flight
    const int LS = p.load_stages;
    const int G = p.K / kGroup;
    auto x_tile = [&](int s) { return smem_base + s * kXBytes; };
    auto wp_tile = [&](int s) { return smem_base + LS * kXBytes + s * kWpBytes; };
    auto wb_tile = [&](int w) { return smem_base + LS * kLoadBytes + w * kWbBytes; };
    const uint32_t scale_base = smem_base + LS * kLoadBytes + kWS * kWbBytes;  // [group][128 rows] fp16
    const uint32_t bar_base = scale_base + G * kBN * 2;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                            // X and packed W have landed
    auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxLoadStages + s); };        // the MMAs that read X have retired
    auto conv_bar = [&](int w) { return bar_base + 8u * (2 * kMaxLoadStages + w); };     // the bf16 weights are written
    auto wfree_bar = [&](int w) { return bar_base + 8u * (2 * kMaxLoadStages + kMaxWbStages + w); };   // ... and read
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kMaxLoadStages + 2 * kMaxWbStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kMaxLoadStages + 2 * kMaxWbStages + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kMaxLoadStages + 2 * kMaxWbStages + 4);
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages_per_tile = p.K / kBK;                  // two per group
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < LS; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int w = 0; w < kWS; ++w) { ptx::mbar_init(conv_bar(w), kConvWarps); ptx::mbar_init(wfree_bar(w), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), kFoldWarps); }
        ptx::fence_mbar_init();
    }
    // rows 128..143 of every stage's B tile: bf16 1.0 in every K position (the swizzle permutes equal chunks)
    for (int i = threadIdx.x; i < (SUB ? 0 : kWS * 16 * 8); i += blockDim.x) {
        const int s = i / 128, r = (i >> 3) & 15, c = i & 7;
        ptx::st_shared_v4(wb_tile(s) + (kBN + r) * 128 + c * 16, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
    }
    ptx::fence_proxy_async_smem();
    if (warp == 1) { ptx::tmem_alloc(tmem_slot, kTmemCols); ptx::tmem_relinquish(); }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            ptx::tma_prefetch_desc(&tmX);
            ptx::tma_prefetch_desc(&tmW);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / p.tiles_n) * kBM, n0 = (tile % p.tiles_n) * kBN;
                for (int i = 0; i < stages_per_tile; ++i) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 31)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(full_bar(stage), kXBytes + kWpBytes);
                    ptx::tma_load_2d(x_tile(stage), &tmX, full_bar(stage), i * kBK, m0);          // x counts bf16 elements
                    ptx::tma_load_2d(wp_tile(stage), &tmW, full_bar(stage), i * (kBK / 2), n0);   // x counts bytes
                    if (++stage == LS) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::umma_idesc(1 /*bf16*/, 1 /*bf16*/, kBM, SUB ? kBN : kBNmma);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            int wst = 0; uint32_t wphase = 0;                       // position in the ring of converted tiles
            int gi = 0;                                             // groups issued so far (over all tiles)
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (int g = 0; g < G && ok; ++g, ++gi) {
                    const int buf = gi & 1;
                    if (!ptx::mbar_wait(tempty_bar(buf), ((gi >> 1) & 1u) ^ 1u, p.status, 32)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * kAccStride;
                    for (int h = 0; h < 2; ++h) {
                        if (!ptx::mbar_wait(full_bar(stage), phase, p.status, 33) ||
                            !ptx::mbar_wait(conv_bar(wst), wphase, p.status, 34)) { ok = false; break; }
                        ptx::tcgen05_fence_after_sync();
                        const uint64_t da = ptx::smem_desc_sw128_kmajor(x_tile(stage)), db = ptx::smem_desc_sw128_kmajor(wb_tile(wst));
#pragma unroll
                        for (int k = 0; k < kBK / 16; ++k)          // 16 K = 32 bytes per instruction: +2 in 16-byte units
                            ptx::umma_f16(d_tmem, da + 2u * k, db + 2u * k, idesc, (h | k) != 0);
                        ptx::umma_commit(empty_bar(stage));
                        ptx::umma_commit(wfree_bar(wst));
                        if (++stage == LS) { stage = 0; phase ^= 1u; }
                        if (++wst == kWS) { wst = 0; wphase ^= 1u; }
                    }
                    if (ok) ptx::umma_commit(tfull_bar(buf));
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp < 2 + kFoldWarps) {
        // ---------------------------------------------------------------- fold: group accumulators -> scaled fp32 sums
        const int q = warp & 3;                                  // TMEM lane quadrant of this warp
        const int half = (warp - 2) >> 2;                        // which 64 of the tile's 128 weight rows
        const int fold_tid = threadIdx.x - 64;
        const __half* sc_sm = reinterpret_cast<const __half*>(smem_gen + (scale_base - smem_base));
        __half* sc_wr = reinterpret_cast<__half*>(smem_gen + (scale_base - smem_base));
        bool ok = true;
        int gi = 0;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile / p.tiles_n) * kBM, n0 = (tile % p.tiles_n) * kBN;
            // the tile's scales, transposed to [group][row] so that a group's 64 scales are eight 16-byte reads
            ptx::named_barrier_1<32 * kFoldWarps>();             // every fold warp is done with the previous tile's scales
            for (int i = fold_tid; i < G * kBN; i += 32 * kFoldWarps) {
                const int r = i & (kBN - 1), g = i >> 7;
                sc_wr[g * kBN + r] = (n0 + r < p.N) ? __ldg(p.S + static_cast<size_t>(n0 + r) * G + g) : __float2half(0.0f);
            }
            ptx::named_barrier_1<32 * kFoldWarps>();
            float acc[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
            for (int g = 0; g < G && ok; ++g, ++gi) {
                const int buf = gi & 1;
                if (!ptx::mbar_wait(tfull_bar(buf), (gi >> 1) & 1u, p.status, 35)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kAccStride;
                uint32_t ones[8] = {};
                if (!SUB) ptx::tmem_ld_32x32b_x8(taddr + kBN, ones);   // sum over the group of this token's activations
                float t = 0.0f;
                constexpr int kCols = 16;                              // accumulator columns per tcgen05.ld
#pragma unroll
                for (int c = 0; c < 64 / kCols; ++c) {                 // registers are the scarce resource
                    uint32_t d[kCols];
                    ptx::tmem_ld_32x32b<kCols>(taddr + 64 * half + kCols * c, d);
                    uint32_t sw[kCols / 2];
#pragma unroll
                    for (int v = 0; v < kCols / 8; ++v) {
                        const uint4 sv = *reinterpret_cast<const uint4*>(sc_sm + g * kBN + 64 * half + kCols * c + 8 * v);
                        sw[4 * v] = sv.x; sw[4 * v + 1] = sv.y; sw[4 * v + 2] = sv.z; sw[4 * v + 3] = sv.w;
                    }
                    ptx::tmem_ld_wait();
                    if (!SUB && c == 0) t = -136.0f * __uint_as_float(ones[0]);
#pragma unroll
                    for (int i = 0; i < kCols / 2; ++i) {
                        const float2 sc2 = __half22float2(*reinterpret_cast<const __half2*>(&sw[i]));
                        float& a0 = acc[kCols * c + 2 * i];
                        float& a1 = acc[kCols * c + 2 * i + 1];
                        if (SUB) {
                            a0 = fmaf(__uint_as_float(d[2 * i]), sc2.x, a0);
                            a1 = fmaf(__uint_as_float(d[2 * i + 1]), sc2.y, a1);
                        } else {
                            a0 = fmaf(__uint_as_float(d[2 * i]) + t, sc2.x, a0);
                            a1 = fmaf(__uint_as_float(d[2 * i + 1]) + t, sc2.y, a1);
                        }
                    }
                }
                ptx::tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(tempty_bar(buf));
            }
            // one rounding to bf16; a thread owns 64 consecutive outputs of its token row
            const int row = m0 + q * 32 + lane;
            if (ok && row < p.M) {
                __nv_bfloat16* dst = p.Y + static_cast<size_t>(row) * p.N + n0 + 64 * half;
                const bool vec = (p.N % 8 == 0) && aligned16(p.Y);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int col = n0 + 64 * half + 8 * j;
                    if (vec && col + 8 <= p.N) {
                        *reinterpret_cast<uint4*>(dst + 8 * j) =
                            make_uint4(pack_bf16x2(acc[8 * j], acc[8 * j + 1]), pack_bf16x2(acc[8 * j + 2], acc[8 * j + 3]),
                                       pack_bf16x2(acc[8 * j + 4], acc[8 * j + 5]), pack_bf16x2(acc[8 * j + 6], acc[8 * j + 7]));
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (col + e < p.N) dst[8 * j + e] = __float2bfloat16_rn(acc[8 * j + e]);
                    }
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- converters: packed int4 -> bf16 B tile
        const int ct = threadIdx.x - 32 * (2 + kFoldWarps);
        const int r = ct & 127;                                  // the weight row this thread converts
        const int team = ct >> 7;
        int stage = 0; uint32_t phase = 0; bool ok = true;
        int wst = 0; uint32_t wphase = 0;
        int it = 0;                                              // running stage index over all tiles
        auto advance = [&]() {
            if (++stage == LS) { stage = 0; phase ^= 1u; }
            if (++wst == kWS) { wst = 0; wphase ^= 1u; }
        };
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (int i = 0; i < stages_per_tile; ++i, ++it) {
                if ((it % kTeams) != team) { advance(); continue; }
                if (!ptx::mbar_wait(full_bar(stage), phase, p.status, 36) ||
                    !ptx::mbar_wait(wfree_bar(wst), wphase ^ 1u, p.status, 37)) { ok = false; break; }
                const uint4* wrow = reinterpret_cast<const uint4*>(smem_gen + (wp_tile(stage) - smem_base) + 32 * r);
                const uint4 w0 = wrow[0], w1 = wrow[1];
                const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {                      // word j: K offsets 8 j .. 8 j + 7 of this stage
                    // nibble pairs (i, i + 4) as bf16 integers 128 + (q + 8): (w & mask) ^ const does the sign flip and
                    // the exponent in one logic operation; then pairs of ascending K by byte permutes
                    uint32_t a0 = (ww[j] & 0x000F000Fu) ^ 0x43084308u;
                    uint32_t a1 = ((ww[j] >> 4) & 0x000F000Fu) ^ 0x43084308u;
                    uint32_t a2 = ((ww[j] >> 8) & 0x000F000Fu) ^ 0x43084308u;
                    uint32_t a3 = ((ww[j] >> 12) & 0x000F000Fu) ^ 0x43084308u;
                    if (SUB) { a0 = sub136(a0); a1 = sub136(a1); a2 = sub136(a2); a3 = sub136(a3); }
                    const int chunk = j ^ (r & 7);                 // 16-byte unit inside the 128-byte row, 128-byte swizzle
                    ptx::st_shared_v4(wb_tile(wst) + r * 128 + chunk * 16, __byte_perm(a0, a1, 0x5410), __byte_perm(a2, a3, 0x5410),
                                      __byte_perm(a0, a1, 0x7632), __byte_perm(a2, a3, 0x7632));
                }
                ptx::fence_proxy_async_smem();                     // the MMA reads these ordinary stores through the async proxy
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(conv_bar(wst));
                advance();
            }
        }
    }

    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace w4p
}  // namespace b200q

namespace b200q {

// Called by b200q_gemm_w4a16 for more than 16 tokens (K a multiple of 128, at most 16384).
int gemm_w4a16_prefill(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int group, int sub, void* stream)
{
    using namespace w4p;
    if (X == nullptr || Wq == nullptr || S == nullptr || Y == nullptr) return cudaErrorInvalidValue;
    if (M <= 0 || N <= 0 || K <= 0 || group != kGroup || K % kGroup != 0 || K / kGroup > kMaxGroups) return cudaErrorInvalidValue;
    if (!aligned16(X) || !aligned16(Wq)) return cudaErrorInvalidValue;
    Params p{};
    p.S = static_cast<const __half*>(S); p.Y = static_cast<__nv_bfloat16*>(Y);
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + kBM - 1) / kBM; p.tiles_n = (N + kBN - 1) / kBN;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    CUtensorMap tmX, tmW;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
        const uint32_t box[2] = {kBK, kBM};
        if (encode_tiled(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    if (!make_tmap_2d_u8(&tmW, Wq, N, K / 2, K / 2, kBN, kBK / 2, CU_TENSOR_MAP_SWIZZLE_NONE)) return cudaErrorInvalidValue;
    const int fixed = 1024 + kBarBytes + 4 * kWbBytes + (K / kGroup) * kBN * 2;
    p.load_stages = (kMaxSmemBytes - fixed) / kLoadBytes;
    if (p.load_stages > kMaxLoadStages) p.load_stages = kMaxLoadStages;
    const int smem_bytes = fixed + p.load_stages * kLoadBytes;
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sms ? tiles : sms;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(w4a16_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemBytes);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(w4a16_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int threads = kThreads + 32 * kConvWarps * (kTeams - 1);
    if (sub) w4a16_prefill_kernel<true><<<grid, threads, smem_bytes, st>>>(tmX, tmW, p);
    else w4a16_prefill_kernel<false><<<grid, threads, smem_bytes, st>>>(tmX, tmW, p);
    return cudaGetLastError();
}

}  // namespace b200q
