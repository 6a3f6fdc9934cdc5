// Block-scaled GEMMs on CTA pairs (tcgen05 cta_group::2): 256 x BN output tile per pair.
//   FMT 0  NVFP4: E2M1 data, one UE4M3 scale per 16 K, kind::mxf4nvf4.block_scale.scale_vec::4X (256 x BN x 64)
//   FMT 1  MXFP8: E4M3 data, one UE8M0 scale per 32 K, kind::mxf8f6f4.block_scale           (256 x BN x 32)
//          (the reference's other block-scaled format: op/test/arch_primitives/ptx_mma_fp8.cu:126-178,
//          scale decoder op/test/arch_primitives/ptx_mma_fp6.cu:344-351)
// Both keep a 128-byte K slab per row and stage and the same blocked scale layout (512-byte blocks of 128
// rows x 4 scales); a block covers 64 K for NVFP4 (one MMA) and 128 K for MXFP8 (four MMAs, which pick their
// scale byte with the scale-factor id of the instruction descriptor).  The text below describes NVFP4.
//
// Same arithmetic and operand formats as gemm_nvfp4.cu (E2M1 data, one UE4M3 scale per 16 K in the
// blocked layout, fp32 accumulate, global scales in the epilogue; formats:
// op/test/arch_primitives/ptx_mma_fp4.cu:49-65,120-144,285-324).  What changes is who loads what:
// each CTA of a pair loads its own 128 rows of A and their scales, HALF of the B tile (BN/2 rows),
// and the scales of the WHOLE B tile (its tensor core multiplies its 128 rows by all BN columns,
// fetching the other half of B from the peer's shared memory).  The B traffic per SM is halved —
// the one-CTA kernel is limited by the L2 -> shared-memory feed at the FP4 rate.
// The leader CTA's MMA thread issues, for both CTAs at once, the scale copies into tensor memory
// (tcgen05.cp.cta_group::2: each CTA copies from its own shared memory into its own TMEM) and the
// MMAs (tcgen05.mma.cta_group::2 kind::mxf4nvf4, 256 x BN x 64).  Barriers as in gemm_fp8_2cta.cuh:
// all loads of both CTAs complete on the leader's "full" barrier (.cta_group::2 loads, no
// multicast), commits with a CTA mask release slots / publish accumulators on both CTAs, the
// epilogue warps of both CTAs (eight per CTA, two per TMEM lane quadrant) release accumulators on the leader's barrier.
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace nvfp4p {

using ptx::tma_load_2d_pair;
using ptx::tma_load_3d_pair;
using ptx::tmem_cp_32x128b_warpx4_pair;
using ptx::umma_mxf4nvf4_pair;
using ptx::umma_mxf8f6f4_pair;

constexpr int kFmtNvfp4 = 0, kFmtMxfp8 = 1;

constexpr int kBM = 128;                 // rows per CTA (256 per pair)
constexpr int kBKBytes = 128;            // per row and stage: 256 E2M1 or 128 E4M3
constexpr int kThreads = 320;            // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue (two per TMEM lane quadrant)
constexpr int kSfBlockBytes = 512;
constexpr uint32_t kTmemCols = 512;

template <int BN, int FMT>
struct Cfg {
    static_assert(BN % 64 == 0 && BN <= 256, "B tile width");
    static constexpr int kBKElems = (FMT == kFmtMxfp8) ? 128 : 256;  // K elements per stage
    static constexpr int kSfBlocks = (FMT == kFmtMxfp8) ? 1 : 4;     // 512-byte scale blocks per row block and stage
    static constexpr int kMaxOff = (BN % 128 == 0) ? 0 : 64;
    static constexpr int kNB = (kMaxOff + BN + 127) / 128;           // scale row-blocks of the whole B tile
    static constexpr int kABytes = kBM * kBKBytes;
    static constexpr int kBHalfBytes = (BN / 2) * kBKBytes;
    static constexpr int kSfaBytes = kSfBlocks * kSfBlockBytes;
    static constexpr int kSfbBytes = kNB * kSfBlocks * kSfBlockBytes;
    static constexpr int kLoadBytes = kABytes + kBHalfBytes + kSfaBytes + kSfbBytes;      // what the TMA loads bring per CTA
    static constexpr int kStageBytes = (kLoadBytes + 1023) / 1024 * 1024;                 // operand tiles start 1024-byte aligned
    static constexpr int kStoreBytes = 8 * 4096;                     // per epilogue warp one 32-row x 64-column bf16 staging buffer
    static constexpr int kStages = (227 * 1024 - 1024 - 256 - kStoreBytes) / kStageBytes > 6 ? 6 : (227 * 1024 - 1024 - 256 - kStoreBytes) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 256;
    static constexpr int kSfCols = 4 * kSfBlocks;                    // TMEM columns of one row block's scales of a stage
    static constexpr int kAccBufs = (2 * BN + kSfCols + kSfCols * kNB <= 512) ? 2 : 1;
    static constexpr int kSfaCol = kAccBufs * BN;
    static constexpr int kSfbCol = kSfaCol + kSfCols;
    static_assert(FMT == kFmtMxfp8 || kLoadBytes % 1024 == 0, "stage alignment");
};

struct Params {
    int M, N, K;
    __nv_bfloat16* C;
    float alpha;
    int tiles_m, tiles_n;
    int group;                   // tile rows (of 256) that walk the N tiles together
    uint32_t* status;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int kGroup, int& tm, int& tn)
{
    const int per_group = kGroup * tiles_n;
    const int g = tile / per_group;
    const int first = g * kGroup;
    const int rows = min(kGroup, tiles_m - first);
    const int r = tile - g * per_group;
    tm = first + r % rows;
    tn = r / rows;
}

template <int BN, int FMT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_nvfp4_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                       const __grid_constant__ CUtensorMap tmC, const Params p)
{
    using C = Cfg<BN, FMT>;
    constexpr int kStages = C::kStages;
    constexpr int kBKElems = C::kBKElems;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t store_base = smem_base + kStages * C::kStageBytes;      // epilogue staging, 1024-byte aligned
    const uint32_t bar_base = store_base + C::kStoreBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - ptx::smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = ptx::cluster_ctarank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int num_kb = (p.K + kBKElems - 1) / kBKElems;
    const int ksteps_total = p.K / (FMT == kFmtMxfp8 ? 32 : 64);     // MMAs along K
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), 16); }
        ptx::fence_mbar_init();
    }
    if (warp == 1) { ptx::tmem_alloc_2cta(tmem_slot, kTmemCols); ptx::tmem_relinquish_2cta(); }
    ptx::tcgen05_fence_before_sync();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        if (ptx::elect_one()) {
            ptx::tma_prefetch_desc(&tmA); ptx::tma_prefetch_desc(&tmB);
            ptx::tma_prefetch_desc(&tmSFA); ptx::tma_prefetch_desc(&tmSFB);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
                int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
                const int m0 = tm * (2 * kBM) + static_cast<int>(cta_rank) * kBM;
                const int n0 = tn * BN;
                const int rb0 = n0 / 128;
                const int mb = m0 / 128;                      // scale row-block of this CTA's A rows
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes, ssfa = sb + C::kBHalfBytes, ssfb = ssfa + C::kSfaBytes;
                    const uint32_t leader_full = ptx::mapa(full_bar(stage), 0);
                    if (cta_rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * C::kLoadBytes);
                    tma_load_2d_pair(sa, &tmA, leader_full, kb * kBKBytes, m0);
                    tma_load_2d_pair(sb, &tmB, leader_full, kb * kBKBytes, n0 + static_cast<int>(cta_rank) * (BN / 2));
                    // scales: the blocked arrays as [row block][K/64 * 2 rows of 256 bytes]; a K slab is 8 such rows,
                    // and one box takes them for all row blocks of the B tile at once
                    tma_load_3d_pair(ssfa, &tmSFA, leader_full, 0, 2 * C::kSfBlocks * kb, mb);
                    tma_load_3d_pair(ssfb, &tmSFB, leader_full, 0, 2 * C::kSfBlocks * kb, rb0);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer (leader only)
        if (cta_rank == 0 && ptx::elect_one()) {
            // NVFP4: E2M1 (format 1 of kind::mxf4nvf4) with UE4M3 scales; MXFP8: E4M3 (format 0 of kind::mxf8f6f4) with
            // UE8M0 scales, scale-factor ids filled in per MMA
            constexpr uint32_t idesc = (FMT == kFmtMxfp8) ? ptx::umma_idesc_block_scaled(0, 0, 2 * kBM, BN, 0, 0, 1)
                                                          : ptx::umma_idesc_block_scaled(1, 1, 2 * kBM, BN, 0, 0, 0);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            int t = 0;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++t) {
                const int buf = (C::kAccBufs == 2) ? (t & 1) : 0;
                const uint32_t par = (C::kAccBufs == 2) ? ((t >> 1) & 1u) : (t & 1u);
                if (!ptx::mbar_wait(tempty_bar(buf), par ^ 1u, p.status, 2)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
                const uint32_t sfb_col_off = ((tn * BN) % 128) / 32;
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, p.status, 3)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const int ksteps = min(4, ksteps_total - 4 * kb);
                    const uint32_t sa = smem_base + stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes, ssfa = sb + C::kBHalfBytes, ssfb = ssfa + C::kSfaBytes;
                    const uint64_t da = ptx::smem_desc_sw128_kmajor(sa), db = ptx::smem_desc_sw128_kmajor(sb);
                    const uint64_t dsfa = ptx::smem_desc_noswizzle_kmajor(ssfa, 16, 128), dsfb = ptx::smem_desc_noswizzle_kmajor(ssfb, 16, 128);
                    const uint32_t tsfa = tmem_base + C::kSfaCol, tsfb = tmem_base + C::kSfbCol;
                    if constexpr (FMT == kFmtMxfp8) {
                        // one scale block per row block serves the four MMAs of the slab: byte ks of every 32-bit scale
                        // column belongs to MMA ks (scale-factor ids in bits [4,6) and [29,31) of the descriptor)
                        tmem_cp_32x128b_warpx4_pair(tsfa, dsfa);
#pragma unroll
                        for (int i = 0; i < C::kNB; ++i) tmem_cp_32x128b_warpx4_pair(tsfb + 4 * i, dsfb + 32u * i);
                        auto kstep = [&](int ks) {
                            const uint32_t id = idesc | (static_cast<uint32_t>(ks) << 4) | (static_cast<uint32_t>(ks) << 29);
                            umma_mxf8f6f4_pair(d_tmem, da + 2u * ks, db + 2u * ks, id, tsfa, tsfb + sfb_col_off, (kb | ks) != 0);
                        };
                        if (ksteps == 4) {
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) kstep(ks);
                        } else {
                            for (int ks = 0; ks < ksteps; ++ks) kstep(ks);
                        }
                    } else {
                        auto kstep = [&](int ks) {
                            // descriptors advance in 16-byte units: one 512-byte scale block = 32
                            tmem_cp_32x128b_warpx4_pair(tsfa + 4 * ks, dsfa + 32u * ks);
#pragma unroll
                            for (int i = 0; i < C::kNB; ++i)
                                tmem_cp_32x128b_warpx4_pair(tsfb + 4 * C::kNB * ks + 4 * i, dsfb + 32u * (i * 4 + ks));
                            umma_mxf4nvf4_pair(d_tmem, da + 2u * ks, db + 2u * ks, idesc, tsfa + 4 * ks,
                                               tsfb + 4 * C::kNB * ks + sfb_col_off, (kb | ks) != 0);
                        };
                        if (ksteps == 4) {
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) kstep(ks);
                        } else {
                            for (int ks = 0; ks < ksteps; ++ks) kstep(ks);
                        }
                    }
                    ptx::umma_commit_2cta(empty_bar(stage), 3);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit_2cta(tfull_bar(buf), 3);
            }
            if (!ok) __nanosleep(200000);
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        // Two warps per TMEM lane quadrant: each owns 32 accumulator rows and up to 128 of the tile's columns.
        // It reads all its columns into registers in one go and hands the accumulator back to the MMA thread
        // (with a single accumulator the tensor pipe idles for exactly this long), then, 64 columns at a
        // time: bf16 into a 128-byte-swizzled staging buffer -> one TMA store of a 32 x 64 box (full 128-byte
        // lines, clipped at the matrix edge by the tensor map).
        const int q = warp & 3;
        const int col_begin = ((warp - 2) >> 2) * 128;                       // first tile column of this warp
        const int nchunks = (min(BN, col_begin + 128) - col_begin) / 64;     // 2, or 1 for the last 64 of a 192-wide tile
        const bool tma_ok = ((static_cast<long long>(p.N) * 2) % 16 == 0) && aligned16(p.C);
        const uint32_t leader_tempty0 = ptx::mapa(tempty_bar(0), 0), leader_tempty1 = ptx::mapa(tempty_bar(1), 0);
        const uint32_t sbuf = store_base + static_cast<uint32_t>(warp - 2) * 4096u;
        const uint64_t store_policy = ptx::l2_policy_evict_first();
        int t = 0; bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++t) {
            const int buf = (C::kAccBufs == 2) ? (t & 1) : 0;
            const uint32_t par = (C::kAccBufs == 2) ? ((t >> 1) & 1u) : (t & 1u);
            int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
            const int row0 = tm * (2 * kBM) + static_cast<int>(cta_rank) * kBM + q * 32;
            const int row = row0 + lane;
            const int n0 = tn * BN + col_begin;
            if (!ptx::mbar_wait(tfull_bar(buf), par, p.status, 4)) { ok = false; break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + col_begin;
            uint32_t r[4][32];
            ptx::tmem_ld_32x32b_x32(taddr, r[0]);
            ptx::tmem_ld_32x32b_x32(taddr + 32, r[1]);
            if (nchunks == 2) {
                ptx::tmem_ld_32x32b_x32(taddr + 64, r[2]);
                ptx::tmem_ld_32x32b_x32(taddr + 96, r[3]);
            }
            ptx::tmem_ld_wait();
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(buf ? leader_tempty1 : leader_tempty0);     // the accumulator is free
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int col0 = n0 + c * 64;
                if (c >= nchunks || row0 >= p.M || col0 >= p.N) continue;
                uint4 o[8];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t (&v)[32] = r[2 * c + h];
                        o[4 * h + i].x = pack_bf16x2(__uint_as_float(v[8 * i + 0]) * p.alpha, __uint_as_float(v[8 * i + 1]) * p.alpha);
                        o[4 * h + i].y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * p.alpha, __uint_as_float(v[8 * i + 3]) * p.alpha);
                        o[4 * h + i].z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * p.alpha, __uint_as_float(v[8 * i + 5]) * p.alpha);
                        o[4 * h + i].w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * p.alpha, __uint_as_float(v[8 * i + 7]) * p.alpha);
                    }
                if (tma_ok) {
                    if (lane == 0) ptx::tma_store_wait_read<0>();      // the store that last read the buffer is done with it
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j)                        // 16-byte unit j of row `lane`, 128-byte swizzle
                        ptx::st_shared_v4(sbuf + lane * 128u + ((j ^ (lane & 7)) << 4), o[j].x, o[j].y, o[j].z, o[j].w);
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) { ptx::tma_store_2d_hint(&tmC, sbuf, col0, row0, store_policy); ptx::tma_store_commit(); }
                } else if (row < p.M) {
                    __nv_bfloat16* dst = p.C + static_cast<size_t>(row) * p.N + col0;
                    const int valid = min(64, p.N - col0);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t w[4] = {o[j].x, o[j].y, o[j].z, o[j].w};
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (8 * j + e < valid)
                                reinterpret_cast<uint16_t*>(dst)[8 * j + e] =
                                    static_cast<uint16_t>((e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xFFFFu));
                    }
                }
            }
        }
        if (lane == 0) ptx::tma_store_wait_all<0>();       // shared memory must outlive the stores that read it
    }

    ptx::tcgen05_fence_before_sync();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc_2cta(tmem_base, kTmemCols);
    }
}

template <int BN, int FMT>
cudaError_t launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmSFA, const CUtensorMap& tmSFB,
                   const CUtensorMap& tmC, Params p, cudaStream_t stream)
{
    auto kernel = gemm_nvfp4_2cta_kernel<BN, FMT>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN, FMT>::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    p.tiles_m = (p.M + 2 * kBM - 1) / (2 * kBM);
    p.tiles_n = (p.N + BN - 1) / BN;
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int tiles = p.tiles_m * p.tiles_n;
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = Cfg<BN, FMT>::kSmemBytes; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmSFA, tmSFB, tmC, p);
}

}  // namespace nvfp4p
}  // namespace b200q

namespace b200q { namespace nvfp4p { int g_group = 0; } }     // 0 = by L2 footprint
extern "C" int b200q_nvfp4_set_group(int g)
{
    if (g < 0 || g > 64) return cudaErrorInvalidValue;
    b200q::nvfp4p::g_group = g;
    return 0;
}
// Called by b200q_gemm_nvfp4_blocked (fmt 0, when the CTA-pair kernel is selected with b200q_nvfp4_set_2cta) and by
// b200q_gemm_mxfp8_blocked (fmt 1).  Operand rows hold K/2 bytes (NVFP4) or K bytes (MXFP8); the blocked scale arrays
// hold one 512-byte block per 128 rows and per 64 K (NVFP4) / 128 K (MXFP8).
namespace b200q {

int gemm_block_scaled_pair(int fmt, const void* Aq, const void* SFA_blocked, const void* Bq, const void* SFB_blocked,
                           void* C, int M, int N, int K, float alpha, int bn, void* stream)
{
    using namespace nvfp4p;
    if (Aq == nullptr || SFA_blocked == nullptr || Bq == nullptr || SFB_blocked == nullptr || C == nullptr)
        return cudaErrorInvalidValue;
    if (fmt != kFmtNvfp4 && fmt != kFmtMxfp8) return cudaErrorInvalidValue;
    if (M <= 0 || N <= 0 || K <= 0 || K % (fmt == kFmtMxfp8 ? 32 : 64) != 0) return cudaErrorInvalidValue;
    if (!aligned16(Aq) || !aligned16(Bq) || !aligned16(SFA_blocked) || !aligned16(SFB_blocked)) return cudaErrorInvalidValue;
    if (bn != 192 && bn != 256) return cudaErrorInvalidValue;
    const size_t row_bytes = fmt == kFmtMxfp8 ? static_cast<size_t>(K) : static_cast<size_t>(K) / 2;
    if (row_bytes % 16 != 0) return cudaErrorInvalidValue;
    Params p{};
    p.M = M; p.N = N; p.K = K; p.C = static_cast<__nv_bfloat16*>(C); p.alpha = alpha;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    p.group = g_group > 0 ? g_group : choose_tile_group((M + 2 * kBM - 1) / (2 * kBM), 2 * kBM, row_bytes);
    CUtensorMap tmA, tmB, tmSFA, tmSFB;
    if (!make_tmap_2d_u8(&tmA, Aq, M, row_bytes, row_bytes, kBM, kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    if (!make_tmap_2d_u8(&tmB, Bq, N, row_bytes, row_bytes, bn / 2, kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    {
        // the blocked scale arrays as [row block][2 * blocks along K][256 bytes]; one box takes the blocks of a
        // K slab for all row blocks of the B tile at once
        const uint64_t blocks_k = fmt == kFmtMxfp8 ? static_cast<uint64_t>((K + 127) / 128) : static_cast<uint64_t>(K / 64);
        const uint32_t slab_rows = fmt == kFmtMxfp8 ? 2u : 8u;
        const uint64_t k_rows = blocks_k * 2;
        const uint64_t strides[2] = {256, k_rows * 256};
        const uint64_t dims_a[3] = {256, k_rows, static_cast<uint64_t>((M + 127) / 128)};
        const uint64_t dims_b[3] = {256, k_rows, static_cast<uint64_t>((N + 127) / 128)};
        const uint32_t box_a[3] = {256, slab_rows, 1};
        const uint32_t box_b[3] = {256, slab_rows, static_cast<uint32_t>(bn == 192 ? Cfg<192, 0>::kNB : Cfg<256, 0>::kNB)};
        if (encode_tiled(&tmSFA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, SFA_blocked, dims_a, strides, box_a, CU_TENSOR_MAP_SWIZZLE_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
        if (encode_tiled(&tmSFB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, SFB_blocked, dims_b, strides, box_b, CU_TENSOR_MAP_SWIZZLE_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    // C as a bf16 matrix with 32-row x 64-column boxes for the epilogue's stores; when N or the pointer rules
    // out a tensor map (row pitch not a multiple of 16 bytes) the kernel stores element-wise and the map is
    // a never-used placeholder over A.
    CUtensorMap tmC = tmA;
    if ((static_cast<long long>(N) * 2) % 16 == 0 && aligned16(C)) {
        const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
        const uint32_t box[2] = {64, 32};
        if (encode_tiled(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (fmt == kFmtMxfp8)
        return bn == 192 ? launch<192, kFmtMxfp8>(tmA, tmB, tmSFA, tmSFB, tmC, p, s) : launch<256, kFmtMxfp8>(tmA, tmB, tmSFA, tmSFB, tmC, p, s);
    return bn == 192 ? launch<192, kFmtNvfp4>(tmA, tmB, tmSFA, tmSFB, tmC, p, s) : launch<256, kFmtNvfp4>(tmA, tmB, tmSFA, tmSFB, tmC, p, s);
}

int gemm_nvfp4_blocked_pair(const void* Aq, const void* SFA_blocked, const void* Bq, const void* SFB_blocked,
                            void* C, int M, int N, int K, float global_a, float global_b, int bn, void* stream)
{
    return gemm_block_scaled_pair(nvfp4p::kFmtNvfp4, Aq, SFA_blocked, Bq, SFB_blocked, C, M, N, K, global_a * global_b, bn, stream);
}
}  // namespace b200q
