// 2:4 structured-sparse FP8 E4M3 GEMM on CTA pairs (tcgen05 cta_group::2): 256 x 224 output tile per pair.
//
// Same operands and arithmetic as gemm_sp24_fp8.cu (Acomp[M,K/2] + Ameta[M,K/8] in the encoding of
// op/test/arch_primitives/ptx_mma_sparse.cu:53-64,163-184; result = dense product with the expanded A,
// ptx_mma_sparse.cu:416-434).  The one-CTA kernel is bound by the L2 -> shared-memory feed of the DENSE B
// operand (48 of the 60 KiB a stage brings in); here each CTA of a pair loads its own 128 rows of compressed
// A with their metadata and HALF of the B tile, and the leader's MMA thread issues
// tcgen05.mma.sp.cta_group::2 (256 x 224 x 64 logical K): both tensor cores read B from both shared memories.
// The metadata boxes go into each CTA's own tensor memory with tcgen05.cp.cta_group::2.128x128b.
// 224 columns: two accumulators fit in tensor memory beside the metadata columns (2 x 224 + 8 <= 512), and
// 4096 x 8192 outputs are exactly 8 waves of 74 pair tiles.  Barriers as in gemm_fp8_2cta.cuh (.cta_group::2
// loads completing on the leader's barrier, no multicast; commits with a CTA mask); epilogue as there
// (swizzled staging + TMA stores).
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace sp24p {

using ptx::tma_load_2d_pair;
using ptx::tmem_cp_128x128b_pair;
using ptx::umma_sp_f8f6f4_pair;

constexpr int kBM = 128;                 // rows per CTA (256 per pair)
constexpr int kBN = 224;                 // tile columns
constexpr int kBKLogical = 256;          // logical K per stage: 128 bytes of compressed A, 256 bytes of B per row
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr int kABytes = kBM * 128;
constexpr int kBHalfTile = (kBN / 2) * 128;              // one 128-logical-K tile of this CTA's B half
constexpr int kMetaBytes = 2 * kBM * 16;                 // two [128][16 B] boxes
constexpr int kStageBytes = kABytes + 2 * kBHalfTile + kMetaBytes;      // 16 + 28 + 4 KiB
constexpr int kStoreBytes = 4 * 2 * 2048;
constexpr int kStages = (227 * 1024 - 1024 - 256 - kStoreBytes) / kStageBytes;
constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 256;
constexpr int kMetaCol = 2 * kBN;                        // metadata columns follow the two accumulators
static_assert(kStageBytes % 1024 == 0 && kStages >= 2 && kMetaCol + 8 <= 512, "tile shape");

struct Params {
    int M, N, K;
    __nv_bfloat16* C;
    float alpha;
    int tiles_m, tiles_n;
    int group;
    int tma_store;
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


__global__ void __launch_bounds__(kThreads, 1)
gemm_sp24_fp8_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmE,
                          const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t store_base = smem_base + kStages * kStageBytes;
    const uint32_t bar_base = store_base + kStoreBytes;
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
    const int num_kb = p.K / kBKLogical + ((p.K % kBKLogical) ? 1 : 0);
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), 8); }
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
            ptx::tma_prefetch_desc(&tmA); ptx::tma_prefetch_desc(&tmE); ptx::tma_prefetch_desc(&tmB);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
                int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
                const int m0 = tm * (2 * kBM) + static_cast<int>(cta_rank) * kBM;
                const int nb = tn * kBN + static_cast<int>(cta_rank) * (kBN / 2);       // this CTA's half of the B tile
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * kStageBytes;
                    const uint32_t sb = sa + kABytes, se = sb + 2 * kBHalfTile;
                    const uint32_t leader_full = ptx::mapa(full_bar(stage), 0);
                    if (cta_rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * kStageBytes);
                    tma_load_2d_pair(sa, &tmA, leader_full, kb * 128, m0);                        // compressed bytes
                    tma_load_2d_pair(sb, &tmB, leader_full, kb * kBKLogical, nb);
                    tma_load_2d_pair(sb + kBHalfTile, &tmB, leader_full, kb * kBKLogical + 128, nb);
                    tma_load_2d_pair(se, &tmE, leader_full, kb * 32, m0);                         // 32 metadata bytes / row
                    tma_load_2d_pair(se + kBM * 16, &tmE, leader_full, kb * 32 + 16, m0);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer (leader only)
        if (cta_rank == 0 && ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::umma_idesc(0, 0, 2 * kBM, kBN, /*sparse=*/true);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            int t = 0;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++t) {
                const int buf = t & 1;
                if (!ptx::mbar_wait(tempty_bar(buf), ((t >> 1) & 1u) ^ 1u, p.status, 2)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * kBN;
                const uint32_t e_tmem = tmem_base + kMetaCol;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, p.status, 3)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t sa = smem_base + stage * kStageBytes;
                    const uint32_t sb = sa + kABytes, se = sb + 2 * kBHalfTile;
                    const uint64_t da = ptx::smem_desc_sw128_kmajor(sa);
                    const int steps = min(4, (p.K - kb * kBKLogical) / 64);
#pragma unroll
                    for (int h = 0; h < 2; ++h)      // metadata of logical K [128h, 128h+128): 4 columns, in both CTAs
                        tmem_cp_128x128b_pair(e_tmem + 4 * h, ptx::smem_desc_noswizzle_kmajor(se + h * kBM * 16, 16, 128));
                    const uint64_t db0 = ptx::smem_desc_sw128_kmajor(sb), db1 = ptx::smem_desc_sw128_kmajor(sb + kBHalfTile);
                    auto kstep = [&](int ks) {
                        umma_sp_f8f6f4_pair(d_tmem, da + 2u * ks, ((ks >> 1) ? db1 : db0) + 4u * (ks & 1), idesc, e_tmem + 2 * ks,
                                            (kb | ks) != 0);
                    };
                    if (steps == 4) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) kstep(ks);
                    } else {
                        for (int ks = 0; ks < steps; ++ks) kstep(ks);
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
        const int q = warp & 3;
        const bool vec_ok = ((static_cast<long long>(p.N) * 2) % 16 == 0) && aligned16(p.C);
        const uint32_t leader_tempty0 = ptx::mapa(tempty_bar(0), 0), leader_tempty1 = ptx::mapa(tempty_bar(1), 0);
        const uint32_t stage_buf = store_base + static_cast<uint32_t>(q) * 4096u;
        const uint64_t store_policy = ptx::l2_policy_evict_first();
        uint32_t chunk_no = 0;
        int t = 0; bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++t) {
            const int buf = t & 1;
            int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
            const int row0 = tm * (2 * kBM) + static_cast<int>(cta_rank) * kBM + q * 32;
            const int row = row0 + lane;
            const int n0 = tn * kBN;
            if (!ptx::mbar_wait(tfull_bar(buf), (t >> 1) & 1u, p.status, 4)) { ok = false; break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kBN;
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
                ptx::tmem_ld_wait();
                if (c == kBN / 32 - 1) {          // last columns read: the accumulator goes back to the MMA thread
                    ptx::tcgen05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive_cluster(buf ? leader_tempty1 : leader_tempty0);
                }
                const int col0 = n0 + c * 32;
                if (row0 >= p.M || col0 >= p.N) continue;
                uint4 o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    o[i].x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * p.alpha, __uint_as_float(r[8 * i + 1]) * p.alpha);
                    o[i].y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * p.alpha, __uint_as_float(r[8 * i + 3]) * p.alpha);
                    o[i].z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * p.alpha, __uint_as_float(r[8 * i + 5]) * p.alpha);
                    o[i].w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * p.alpha, __uint_as_float(r[8 * i + 7]) * p.alpha);
                }
                if (p.tma_store) {
                    const uint32_t sbuf = stage_buf + (chunk_no & 1u) * 2048u;
                    ++chunk_no;
                    if (lane == 0) ptx::tma_store_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t off = lane * 64u + j * 16u;
                        const uint32_t phys = off ^ (((off >> 7) & 3u) << 4);           // 64-byte swizzle
                        ptx::st_shared_v4(sbuf + phys, o[j].x, o[j].y, o[j].z, o[j].w);
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) { ptx::tma_store_2d_hint(&tmC, sbuf, col0, row0, store_policy); ptx::tma_store_commit(); }
                } else if (row < p.M) {
                    __nv_bfloat16* dst = p.C + static_cast<size_t>(row) * p.N + col0;
                    const int valid = min(32, p.N - col0);
                    if (vec_ok && valid == 32) {
                        uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
                        for (int i = 0; i < 4; ++i) d[i] = o[i];
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]) * p.alpha);
                    }
                }
            }
        }
        if (lane == 0) ptx::tma_store_wait_all<0>();
    }

    ptx::tcgen05_fence_before_sync();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc_2cta(tmem_base, kTmemCols);
    }
}

}  // namespace sp24p

// Called by b200q_gemm_sp24_fp8 when the CTA-pair kernel is selected (b200q_sp24_set_2cta) and M > 128.
int gemm_sp24_fp8_pair(const void* Acomp, const void* Ameta, const void* B, void* C, int M, int N, int K, float alpha, void* stream)
{
    using namespace sp24p;
    Params p{};
    p.M = M; p.N = N; p.K = K; p.C = static_cast<__nv_bfloat16*>(C); p.alpha = alpha;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    p.tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
    p.tiles_n = (N + kBN - 1) / kBN;
    p.group = choose_tile_group(p.tiles_m, 2 * kBM, static_cast<size_t>(K) / 2);
    CUtensorMap tmA, tmE, tmB;
    if (!make_tmap_2d_u8(&tmA, Acomp, M, K / 2, K / 2, kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    if (!make_tmap_2d_u8(&tmE, Ameta, M, K / 8, K / 8, kBM, 16, CU_TENSOR_MAP_SWIZZLE_NONE)) return cudaErrorInvalidValue;
    if (!make_tmap_2d_u8(&tmB, B, N, K, K, kBN / 2, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    CUtensorMap tmC = tmA;
    p.tma_store = 0;
    if ((static_cast<long long>(N) * 2) % 16 == 0 && aligned16(C)) {
        const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
        const uint32_t box[2] = {32, 32};
        if (encode_tiled(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
        p.tma_store = 1;
    }
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(gemm_sp24_fp8_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int tiles = p.tiles_m * p.tiles_n;
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes; cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_sp24_fp8_2cta_kernel, tmA, tmE, tmB, tmC, p);
}

}  // namespace b200q
