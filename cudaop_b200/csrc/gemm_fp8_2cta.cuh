// FP8 E4M3 GEMM on CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs on neighbouring SMs
// computes one 256 x 256 output tile per step.
//
// Each CTA loads its own 128 rows of A and ITS HALF (128 rows) of the B tile — half the B traffic
// per SM of the one-CTA kernel, which is what bounds that kernel (L2 -> shared memory) — and the
// leader CTA's single MMA thread issues tcgen05.mma.cta_group::2 (256 x 256 x 32): the tensor cores
// of both SMs read A from their own shared memory and B from both, and each accumulates its 128
// rows in its own tensor memory.  Synchronisation across the pair:
//   * both producers' TMA loads (cp.async.bulk.tensor ... .cta_group::2, no multicast) complete on the
//     LEADER's "full" barrier, for which the leader's producer posts the byte count of both CTAs;
//   * tcgen05.commit.cta_group::2 with a CTA mask releases the ring slot ("empty") and publishes the
//     accumulator ("tmem full") on both CTAs at once (a signal multicast, not a data load);
//   * the epilogue warps of both CTAs hand accumulator buffers back by arriving on the leader's
//     "tmem empty" barrier (the peer through the cluster address of that barrier).
// bf16 results leave through shared memory: each epilogue warp packs 32 rows x kCW columns into a
// swizzled staging buffer and one lane issues a TMA store of that box (whole 32/64-byte row pieces
// per request instead of 16 bytes per thread; the tensor map clips at the matrix edge).
// With the SwiGLU epilogue the leader's B half is the gate rows and the peer's the up rows, so every
// CTA again holds gate | up of its 128 token rows side by side.
// Tile scheduling: the leader's producer thread decides which tile the pair does next and publishes the number
// in a 16-entry ring in both CTAs' shared memory (a DSMEM store for the peer) behind one mbarrier per entry;
// every other role of both CTAs reads the ring.  With a scheduler slot (Params::sched) the number comes from a
// global atomic counter, fetched one tile ahead so its latency is hidden: a pair that is slowed down — by another
// kernel sharing its SMs, such as the all-reduce of the previous step — simply takes fewer tiles instead of
// holding the whole grid up with a fixed share.  The last pair to finish resets the slot for the next launch.
// Without a slot the sequence is the static pair, pair + pairs, ...
#pragma once
#include <type_traits>

#include "gemm_fp8.cuh"

namespace b200q {
namespace fp8 {

using ptx::tma_load_2d_pair;

constexpr int kPairBM = 256;
template <int BN>
struct PairCfg {
    static constexpr int kBHalfRows = BN / 2;                           // B rows each CTA loads
    static constexpr int kStageBytes = kBM * kBK + kBHalfRows * kBK;    // A 16 KiB + B half (16 or 14 KiB)
    static constexpr int kStages = 6;
    static constexpr int kStoreBytes = 4 * 2 * 2048;                    // per epilogue warp two 32-row x 64-byte staging buffers
    static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 512;    // + alignment slack + barriers and tile ring
    static_assert(kStageBytes % 1024 == 0 && BN % 32 == 0, "tile shape");
};


template <int EPI, typename OutT, int BN>
__global__ void __launch_bounds__(kBaseThreads, 1)
gemm_fp8_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmC, const Params p)
{
    using PC = PairCfg<BN>;
    constexpr int kStages = PC::kStages;
    constexpr int kPairStageBytes = PC::kStageBytes;
    constexpr int kPairBN = BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t store_base = smem_base + kStages * kPairStageBytes;     // epilogue staging (1024-byte aligned)
    const uint32_t bar_base = store_base + PC::kStoreBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - ptx::smem_u32(smem_raw)));
    constexpr int kRing = 16;
    auto sched_bar = [&](int i) { return bar_base + 8u * (2 * kStages + 5 + i); };     // tile-ring entry i has been written
    const uint32_t ring = bar_base + 8u * (2 * kStages + 5 + kRing);                    // kRing tile numbers
    volatile int* ring_ptr = reinterpret_cast<volatile int*>(smem_raw + (ring - ptx::smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = ptx::cluster_ctarank();          // 0 = leader of the pair
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int num_kb = (p.K + kBK - 1) / kBK;
    const int num_tiles = p.tiles_m * p.tiles_n;                // 256-row x 256-column (SwiGLU: 128 output columns) tiles
    constexpr int kOutCols = (EPI == kEpiSwiGLU) ? BN / 2 : BN;
    constexpr int kCW = (kOutCols % 32 == 0) ? 32 : 16;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), 8); }
        for (int i = 0; i < kRing; ++i) ptx::mbar_init(sched_bar(i), 1);
        ptx::fence_mbar_init();
    }
    // The t-th tile of this pair, as published by the leader's producer (>= num_tiles: no more).  An entry is
    // overwritten kRing tiles later, when every reader is past it: the leader's producer is at most kStages K-blocks
    // (with a short K: that many tiles) ahead of the peer's producer and of the MMA thread, which is at most two
    // accumulators ahead of the epilogue — nine tiles at the very most.
    static_assert(kRing >= kStages + 4, "tile ring depth");
    auto tile_at = [&](int t, uint32_t site, bool& ok) -> int {
        if (!ptx::mbar_wait(sched_bar(t & (kRing - 1)), (t / kRing) & 1u, p.status, site)) { ok = false; return num_tiles; }
        return ring_ptr[t & (kRing - 1)];
    };
    if (warp == 1) { ptx::tmem_alloc_2cta(tmem_slot, kTmemCols); ptx::tmem_relinquish_2cta(); }
    ptx::tcgen05_fence_before_sync();
    ptx::cluster_arrive();          // both CTAs' barriers are initialised before anyone signals across the pair
    ptx::cluster_wait();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (ptx::elect_one()) {
            ptx::tma_prefetch_desc(&tmA);
            ptx::tma_prefetch_desc(&tmB);
            if (EPI == kEpiSwiGLU) ptx::tma_prefetch_desc(&tmB2);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            int static_next = pair;
            auto fetch = [&]() -> int {                     // leader only: the next tile of this pair
                if (p.sched != nullptr) return static_cast<int>(atomicAdd(p.sched, 1u));
                const int t = static_next; static_next += pairs; return t;
            };
            int ahead = (cta_rank == 0) ? fetch() : 0;
            for (int t = 0; ok; ++t) {
                int tile;
                if (cta_rank == 0) {
                    tile = ahead < num_tiles ? ahead : num_tiles;
                    const int e = t & (kRing - 1);
                    ring_ptr[e] = tile;
                    ptx::st_shared_cluster_u32(ptx::mapa(ring + 4u * e, 1), static_cast<uint32_t>(tile));
                    ptx::mbar_arrive(sched_bar(e));
                    ptx::mbar_arrive_cluster(ptx::mapa(sched_bar(e), 1));           // release: the peer sees the entry
                    if (tile < num_tiles) ahead = fetch();                          // for the next round; not waited for here
                } else {
                    tile = tile_at(t, 9, ok);
                }
                if (tile >= num_tiles) break;
                int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
                const int m0 = tm * kPairBM + static_cast<int>(cta_rank) * kBM;
                const int n0 = tn * kOutCols;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * kPairStageBytes, sb = sa + kBM * kBK;
                    const uint32_t leader_full = ptx::mapa(full_bar(stage), 0);
                    if (cta_rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * kPairStageBytes);   // bytes of both CTAs
                    tma_load_2d_pair(sa, &tmA, leader_full, kb * kBK, m0);
                    if (EPI == kEpiSwiGLU) {       // leader: gate rows, peer: up rows
                        tma_load_2d_pair(sb, cta_rank == 0 ? &tmB : &tmB2, leader_full, kb * kBK, n0);
                    } else {
                        tma_load_2d_pair(sb, &tmB, leader_full, kb * kBK, n0 + static_cast<int>(cta_rank) * (BN / 2));
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            // dynamic scheduling: every pair fetched exactly one number >= num_tiles (or gave up); the last pair to get
            // here leaves the slot zeroed for the next launch on this stream
            if (cta_rank == 0 && p.sched != nullptr) {
                if (!ok) { while (ahead < num_tiles) ahead = fetch(); }          // drain, so that every pair's last fetch is a terminating one
                __threadfence();
                if (atomicAdd(p.sched + 1, 1u) + 1u == static_cast<uint32_t>(pairs)) { p.sched[0] = 0u; p.sched[1] = 0u; __threadfence(); }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer (leader CTA only)
        if (cta_rank == 0 && ptx::elect_one()) {
            constexpr uint32_t idesc = (EPI == kEpiInt32) ? ptx::umma_idesc_i8(kPairBM, kPairBN) : ptx::umma_idesc(0, 0, kPairBM, kPairBN);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int t = 0; ok; ++t) {
                if (tile_at(t, 10, ok) >= num_tiles) break;
                const int buf = t & 1;
                if (!ptx::mbar_wait(tempty_bar(buf), ((t >> 1) & 1u) ^ 1u, p.status, 2)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * 256;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, p.status, 3)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t sa = smem_base + stage * kPairStageBytes, sb = sa + kBM * kBK;
                    const uint64_t da = ptx::smem_desc_sw128_kmajor(sa), db = ptx::smem_desc_sw128_kmajor(sb);
#pragma unroll
                    for (int k = 0; k < kBK / 32; ++k) {
                        if (EPI == kEpiInt32) ptx::umma_i8_2cta(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0);
                        else ptx::umma_f8f6f4_2cta(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0);
                    }
                    ptx::umma_commit_2cta(empty_bar(stage), 3);        // slot free on both CTAs
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit_2cta(tfull_bar(buf), 3);      // accumulator ready on both CTAs
            }
            if (!ok) __nanosleep(200000);
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
        const int q = warp & 3;
        OutT* Cbase = static_cast<OutT*>(p.C);
        const bool ld_ok = ((p.ldc * (long long)sizeof(OutT)) % 16 == 0) && aligned16(p.C);
        const uint32_t leader_tempty0 = ptx::mapa(tempty_bar(0), 0), leader_tempty1 = ptx::mapa(tempty_bar(1), 0);
        constexpr bool kBf16Out = std::is_same<OutT, __nv_bfloat16>::value;
        constexpr uint32_t kRowBytes = kCW * 2;                // staging row: 64 or 32 bytes, swizzled over that span
        constexpr uint32_t kSwzMask = kRowBytes / 16 - 1;
        const bool tma_store = kBf16Out && p.tma_store != 0;
        const uint32_t stage_buf = store_base + static_cast<uint32_t>(q) * 4096u;
        const uint64_t store_policy = ptx::l2_policy_evict_first();
        uint32_t chunk_no = 0;
        bool ok = true;
        for (int t = 0; ok; ++t) {
            const int tile = tile_at(t, 11, ok);
            if (tile >= num_tiles) break;
            const int buf = t & 1;
            int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
            const int row = tm * kPairBM + static_cast<int>(cta_rank) * kBM + q * 32 + lane;
            const int n0 = tn * kOutCols;
            if (!ptx::mbar_wait(tfull_bar(buf), (t >> 1) & 1u, p.status, 4)) { ok = false; break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * 256;
            float rs = 1.0f;
            if (EPI == kEpiRowCol || EPI == kEpiSwiGLU) rs = (row < p.M) ? __ldg(p.row_scale + row) : 0.0f;
#pragma unroll 1
            for (int c = 0; c < kOutCols / kCW; ++c) {
                uint32_t r[kCW];
                float v[kCW];
                const int col0 = n0 + c * kCW;
                ptx::tmem_ld_32x32b<kCW>(taddr + c * kCW, r);
                if (EPI == kEpiSwiGLU) {
                    uint32_t ru[kCW];
                    ptx::tmem_ld_32x32b<kCW>(taddr + BN / 2 + c * kCW, ru);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < kCW; ++i) {
                        const int col = col0 + i;
                        const float sg = (col < p.N) ? __ldg(p.col_scale + col) : 0.0f;
                        const float su = (col < p.N) ? __ldg(p.col_scale2 + col) : 0.0f;
                        const float g = __uint_as_float(r[i]) * (rs * sg);
                        const float u = __uint_as_float(ru[i]) * (rs * su);
                        v[i] = g / (1.0f + __expf(-g)) * u;
                    }
                } else if (EPI == kEpiInt32) {
                    // the accumulator is a 32-bit integer: pass its bits through (plus the optional addend, wrapping)
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < kCW; ++i) {
                        uint32_t acc = r[i];
                        if (p.c_in != nullptr && row < p.M && col0 + i < p.N)
                            acc += static_cast<uint32_t>(__ldg(p.c_in + (long long)row * p.ldc + col0 + i));
                        v[i] = __uint_as_float(acc);
                    }
                } else {
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < kCW; ++i) {
                        float s;
                        if (EPI == kEpiTensor) s = p.alpha;
                        else { const int col = col0 + i; s = rs * ((col < p.N) ? __ldg(p.col_scale + col) : 0.0f); }
                        v[i] = __uint_as_float(r[i]) * s;
                    }
                }
                if (tma_store) {
                    if constexpr (kBf16Out) {
                        const int row0 = row - lane;
                        if (row0 < p.M && col0 < p.N) {
                            const uint32_t sbuf = stage_buf + (chunk_no & 1u) * 2048u;
                            ++chunk_no;
                            if (lane == 0) ptx::tma_store_wait_read<1>();     // the store that last read this buffer has finished reading
                            __syncwarp();
#pragma unroll
                            for (int j = 0; j < kCW / 8; ++j) {
                                const uint32_t off = lane * kRowBytes + j * 16u;
                                const uint32_t phys = off ^ (((off >> 7) & kSwzMask) << 4);
                                ptx::st_shared_v4(sbuf + phys, pack_bf16x2(v[8 * j + 0], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                                                 pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
                            }
                            ptx::fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) { ptx::tma_store_2d_hint(&tmC, sbuf, col0, row0, store_policy); ptx::tma_store_commit(); }
                        }
                    }
                } else if (row < p.M && col0 < p.N) {
                    const int valid = min(kCW, p.N - col0);
                    OutPack<OutT>::template store<kCW>(Cbase + (long long)row * p.ldc + col0, v, ld_ok && valid == kCW, valid);
                }
            }
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(buf ? leader_tempty1 : leader_tempty0);
        }
        if (lane == 0) ptx::tma_store_wait_all<0>();      // shared memory must outlive the stores that read it
    }

    // both CTAs are done with tensor memory (every accumulator was drained) before either frees it
    ptx::tcgen05_fence_before_sync();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc_2cta(tmem_base, kTmemCols);
    }
}

}  // namespace fp8
}  // namespace b200q
