// 2:4 structured-sparse FP8 E4M3 GEMM for sm_100a:
//   C[M,N] (bf16) = ( expand(Acomp, Ameta) * B^T ) * (scale_a * scale_b)
// Acomp[M,K/2] keeps the two retained values of every four consecutive K in order; Ameta[M,K/8]
// holds one nibble per group of four — two ascending 2-bit positions, lower position in bits
// [1:0], nibbles packed low-first — exactly the encoding of
// op/test/arch_primitives/ptx_mma_sparse.cu:53-64,163-184.  The result is the dense product with the
// expanded A (the reference's ground truth, ptx_mma_sparse.cu:416-434).
//
// Kernel: the FP8 kernel's structure with tcgen05.mma.sp kind::f8f6f4 (128 x BN x 64 logical K per
// instruction: 32 bytes of compressed A, 64 bytes of B per row).  A stage holds 256 logical K:
// one 128-byte-swizzled tile of compressed A, two 128-byte-swizzled tiles of B, and the metadata
// of the slab as two [128 rows][16 bytes] boxes that TMA cuts straight out of the row-major Ameta
// (one bit per logical element).  The issuing thread copies each box into four TMEM columns
// (tcgen05.cp 128x128b) ahead of the two MMAs that read it (two columns each).
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace sp24 {

constexpr int kBM = 128;
constexpr int kBKLogical = 256;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;

template <int BN>
struct Cfg {
    static constexpr int kABytes = kBM * 128;            // compressed A: 128 bytes = 256 logical K per row
    static constexpr int kBHalf = BN * 128;              // one 128-logical-K tile of B
    static constexpr int kMetaBytes = 2 * kBM * 16;      // two [128][16 B] boxes
    static constexpr int kStageBytes = kABytes + 2 * kBHalf + kMetaBytes;
    static constexpr int kStoreBytes = 4 * 2 * 2048;     // per epilogue warp two 32-row x 32-column bf16 staging buffers
    static constexpr int kStages = (227 * 1024 - 1024 - 256 - kStoreBytes) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 256;
    static constexpr int kAccBufs = 2 * BN + 8 <= 512 ? 2 : 1;
    static constexpr int kMetaCol = kAccBufs * BN;
    static_assert(kStageBytes % 1024 == 0, "stage alignment");
    static_assert(kStages >= 2, "need at least two stages");
};

struct Params {
    int M, N, K;
    __nv_bfloat16* C;
    float alpha;
    int tiles_m, tiles_n;
    int group;                   // tile rows that walk the N tiles together
    int tma_store;               // bf16 results leave through TMA stores (tensor map valid)
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

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_sp24_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmE,
                     const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC, const Params p)
{
    using C = Cfg<BN>;
    constexpr int kStages = C::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t store_base = smem_base + kStages * C::kStageBytes;      // epilogue staging (1024-byte aligned)
    const uint32_t bar_base = store_base + C::kStoreBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - ptx::smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = p.K / kBKLogical + ((p.K % kBKLogical) ? 1 : 0);
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), 4); }
        ptx::fence_mbar_init();
    }
    if (warp == 1) { ptx::tmem_alloc(tmem_slot, kTmemCols); ptx::tmem_relinquish(); }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        if (ptx::elect_one()) {
            ptx::tma_prefetch_desc(&tmA); ptx::tma_prefetch_desc(&tmE); ptx::tma_prefetch_desc(&tmB);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
                const int m0 = tm * kBM, n0 = tn * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes, se = sb + 2 * C::kBHalf;
                    ptx::mbar_arrive_expect_tx(full_bar(stage), C::kStageBytes);
                    ptx::tma_load_2d(sa, &tmA, full_bar(stage), kb * 128, m0);                    // compressed bytes
                    ptx::tma_load_2d(sb, &tmB, full_bar(stage), kb * kBKLogical, n0);
                    ptx::tma_load_2d(sb + C::kBHalf, &tmB, full_bar(stage), kb * kBKLogical + 128, n0);
                    ptx::tma_load_2d(se, &tmE, full_bar(stage), kb * 32, m0);                     // 32 metadata bytes / row
                    ptx::tma_load_2d(se + kBM * 16, &tmE, full_bar(stage), kb * 32 + 16, m0);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp == 1) {
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::umma_idesc(0, 0, kBM, BN, /*sparse=*/true);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            int t = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
                const int buf = (C::kAccBufs == 2) ? (t & 1) : 0;
                const uint32_t par = (C::kAccBufs == 2) ? ((t >> 1) & 1u) : (t & 1u);
                if (!ptx::mbar_wait(tempty_bar(buf), par ^ 1u, p.status, 2)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const uint32_t e_tmem = tmem_base + C::kMetaCol;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, p.status, 3)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t sa = smem_base + stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes, se = sb + 2 * C::kBHalf;
                    const uint64_t da = ptx::smem_desc_sw128_kmajor(sa);
                    const int steps = min(4, (p.K - kb * kBKLogical) / 64);
#pragma unroll
                    for (int h = 0; h < 2; ++h)      // metadata of logical K [128h, 128h+128): 4 columns
                        ptx::tmem_cp_128x128b(e_tmem + 4 * h, ptx::smem_desc_noswizzle_kmajor(se + h * kBM * 16, 16, 128));
                    const uint64_t db0 = ptx::smem_desc_sw128_kmajor(sb), db1 = ptx::smem_desc_sw128_kmajor(sb + C::kBHalf);
                    auto kstep = [&](int ks) {
                        ptx::umma_sp_f8f6f4(d_tmem, da + 2u * ks, ((ks >> 1) ? db1 : db0) + 4u * (ks & 1), idesc, e_tmem + 2 * ks,
                                            (kb | ks) != 0);
                    };
                    if (steps == 4) {                // the single issuing thread is on the critical path: no loop overhead
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) kstep(ks);
                    } else {
                        for (int ks = 0; ks < steps; ++ks) kstep(ks);
                    }
                    ptx::umma_commit(empty_bar(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit(tfull_bar(buf));
            }
            if (!ok) __nanosleep(200000);
        }
    } else {
        // Each warp owns 32 accumulator rows; 32 columns at a time: tensor memory -> registers -> bf16 in a
        // 64-byte-swizzled staging buffer -> one TMA store of the 32 x 32 box (clipped at the matrix edge by the
        // tensor map, evict-first in L2).  Without a usable tensor map: 16-byte stores per thread.
        const int q = warp & 3;
        const bool vec_ok = ((static_cast<long long>(p.N) * 2) % 16 == 0) && aligned16(p.C);
        const uint32_t stage_buf = store_base + static_cast<uint32_t>(q) * 4096u;
        const uint64_t store_policy = ptx::l2_policy_evict_first();
        uint32_t chunk_no = 0;
        int t = 0; bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
            const int buf = (C::kAccBufs == 2) ? (t & 1) : 0;
            const uint32_t par = (C::kAccBufs == 2) ? ((t >> 1) & 1u) : (t & 1u);
            int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
            const int row0 = tm * kBM + q * 32;
            const int row = row0 + lane;
            const int n0 = tn * BN;
            if (!ptx::mbar_wait(tfull_bar(buf), par, p.status, 4)) { ok = false; break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
                ptx::tmem_ld_wait();
                if (c == BN / 32 - 1) {           // last columns read: the accumulator goes back to the MMA thread
                    ptx::tcgen05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(tempty_bar(buf));
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
                    if (lane == 0) ptx::tma_store_wait_read<1>();     // the store that last read this buffer has finished reading
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
        if (lane == 0) ptx::tma_store_wait_all<0>();       // shared memory must outlive the stores that read it
    }

    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int BN>
cudaError_t launch(const CUtensorMap& tmA, const CUtensorMap& tmE, const CUtensorMap& tmB, const CUtensorMap& tmC, Params p,
                   cudaStream_t stream)
{
    auto kernel = gemm_sp24_fp8_kernel<BN>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    p.tiles_m = (p.M + kBM - 1) / kBM;
    p.tiles_n = (p.N + BN - 1) / BN;
    p.group = choose_tile_group(p.tiles_m, kBM, static_cast<size_t>(p.K) / 2);     // compressed A rows of a group stay in L2
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int tiles = p.tiles_m * p.tiles_n;
    kernel<<<tiles < sms ? tiles : sms, kThreads, Cfg<BN>::kSmemBytes, stream>>>(tmA, tmE, tmB, tmC, p);
    return cudaGetLastError();
}

int g_tile_n = 192;
int g_use_2cta = 1;      // 1 (default): CTA-pair kernel (gemm_sp24_fp8_2cta.cu, 256 x 224 tiles) for M > 128 (b200q_sp24_set_2cta)

}  // namespace sp24
}  // namespace b200q

namespace b200q {
// gemm_sp24_fp8_2cta.cu
int gemm_sp24_fp8_pair(const void* Acomp, const void* Ameta, const void* B, void* C, int M, int N, int K, float alpha, void* stream);
}

extern "C" {

int b200q_sp24_set_2cta(int on)
{
    b200q::sp24::g_use_2cta = on ? 1 : 0;
    return 0;
}

int b200q_sp24_set_tile_n(int bn)
{
    if (bn != 128 && bn != 192 && bn != 256) return cudaErrorInvalidValue;
    b200q::sp24::g_tile_n = bn;
    return 0;
}

int b200q_gemm_sp24_fp8(const void* Acomp, const void* Ameta, const void* B, void* C, int M, int N, int K,
                        float scale_a, float scale_b, void* stream)
{
    using namespace b200q;
    if (Acomp == nullptr || Ameta == nullptr || B == nullptr || C == nullptr) return cudaErrorInvalidValue;
    if (M <= 0 || N <= 0 || K <= 0 || K % 128 != 0) return cudaErrorInvalidValue;
    if (!aligned16(Acomp) || !aligned16(Ameta) || !aligned16(B)) return cudaErrorInvalidValue;
    if (sp24::g_use_2cta && M > sp24::kBM) return gemm_sp24_fp8_pair(Acomp, Ameta, B, C, M, N, K, scale_a * scale_b, stream);
    sp24::Params p{};
    p.M = M; p.N = N; p.K = K; p.C = static_cast<__nv_bfloat16*>(C); p.alpha = scale_a * scale_b;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    const int bn = sp24::g_tile_n;
    CUtensorMap tmA, tmE, tmB;
    if (!make_tmap_2d_u8(&tmA, Acomp, M, K / 2, K / 2, sp24::kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    if (!make_tmap_2d_u8(&tmE, Ameta, M, K / 8, K / 8, sp24::kBM, 16, CU_TENSOR_MAP_SWIZZLE_NONE)) return cudaErrorInvalidValue;
    if (!make_tmap_2d_u8(&tmB, B, N, K, K, bn, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    // C as a bf16 matrix with the epilogue's 32 x 32 boxes; a row pitch that is not a multiple of 16 bytes rules the
    // tensor map out, and the kernel then stores from registers
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
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (bn == 128) return sp24::launch<128>(tmA, tmE, tmB, tmC, p, s);
    if (bn == 256) return sp24::launch<256>(tmA, tmE, tmB, tmC, p, s);
    return sp24::launch<192>(tmA, tmE, tmB, tmC, p, s);
}

}  // extern "C"
