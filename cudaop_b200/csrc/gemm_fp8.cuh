// FP8 E4M3 GEMM for sm_100a:  C[M,N] = epilogue( A[M,K] * B[N,K]^T ), fp32 accumulate.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0    TMA producer  : 128-byte-swizzled A (128 x 128 B) and B (256 x 128 B) tiles into a
//                             4-stage shared-memory ring, completion on "full" mbarriers
//   warp 1    MMA issuer    : one elected thread issues tcgen05.mma kind::f8f6f4 (128 x 256 x 32)
//                             reading shared memory through matrix descriptors, accumulating into
//                             TMEM; tcgen05.commit releases ring slots and publishes accumulators
//   warps 2-5 epilogue      : tcgen05.ld the 128 x 256 fp32 accumulator (one TMEM lane = one row),
//                             apply the scale rule, cast to the output type, 16-byte stores
// TMEM holds two accumulators (2 x 256 columns), so the epilogue of tile i overlaps the
// main loop of tile i+1.  No cluster, no multicast.
//
// Semantics follow the reference: operands K-contiguous, C = A * B^T (op/cpu/cpu_ops.cpp:95-113);
// per-tensor scales are not MMA operands, the epilogue multiplies the fp32 accumulator
// (op/test/arch_primitives/ptx_mma_fp8.cu:16-23); the output cast is round-to-nearest-even from
// fp32 at the very end (op/test/arch_primitives/ptx_mma_fp4.cu:277-282).
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace b200q {
namespace fp8 {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 128;           // bytes == elements for FP8: one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kABytes = kBM * kBK;                 // 16 KiB
constexpr int kBBytes = kBN * kBK;                 // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;     // 48 KiB
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr uint32_t kTmemCols = 512;

enum Epilogue : int {
    kEpiTensor = 0,   // C = acc * alpha                                  (per-tensor scales)
    kEpiRowCol = 1,   // C = acc * (row_scale[m] * col_scale[n])          (per-token x per-channel)
    kEpiSwiGLU = 2,   // B tile = 128 gate rows + 128 up rows; C[m,n] = silu(g) * u, 128 columns per tile
};

struct Params {
    int M, N, K;                 // N = number of OUTPUT columns
    void* C;
    long long ldc;               // elements
    float alpha;
    const float* row_scale;      // [M]
    const float* col_scale;      // [N]   (gate scales for SwiGLU)
    const float* col_scale2;     // [N]   (up scales for SwiGLU)
    int tiles_m, tiles_n;
    uint32_t* status;
};

template <typename OutT> struct OutPack;
template <> struct OutPack<__nv_bfloat16> {
    // 32 fp32 -> 32 bf16 = 64 bytes
    static __device__ __forceinline__ void store32(__nv_bfloat16* dst, const float (&v)[32], bool vec, int valid)
    {
        if (vec) {
            uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 q;
                q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
                q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
                q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
                q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
                d[i] = q;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i < valid) dst[i] = __float2bfloat16_rn(v[i]);
        }
    }
};
template <> struct OutPack<float> {
    static __device__ __forceinline__ void store32(float* dst, const float (&v)[32], bool vec, int valid)
    {
        if (vec) {
            float4* d = reinterpret_cast<float4*>(dst);
#pragma unroll
            for (int i = 0; i < 8; ++i) d[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i < valid) dst[i] = v[i];
        }
    }
};

// Tile order: groups of 16 tile-rows walk the N tiles together so that the CTAs running
// at the same time share A and B tiles in L2.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn)
{
    constexpr int kGroup = 16;
    const int per_group = kGroup * tiles_n;
    const int g = tile / per_group;
    const int first = g * kGroup;
    const int rows = min(kGroup, tiles_m - first);
    const int r = tile - g * per_group;
    tm = first + r % rows;
    tn = r / rows;
}

template <int EPI, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmB2, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + kStages * kStageBytes;
    // barrier layout (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], then tmem ptr
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - ptx::smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_kb = (p.K + kBK - 1) / kBK;
    const int num_tiles = p.tiles_m * p.tiles_n;
    constexpr int kOutCols = (EPI == kEpiSwiGLU) ? 128 : kBN;   // output columns per tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), 4); }
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            ptx::tma_prefetch_desc(&tmA);
            ptx::tma_prefetch_desc(&tmB);
            if (EPI == kEpiSwiGLU) ptx::tma_prefetch_desc(&tmB2);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                const int m0 = tm * kBM, n0 = tn * kOutCols;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * kStageBytes, sb = sa + kABytes;
                    ptx::mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
                    ptx::tma_load_2d(sa, &tmA, full_bar(stage), kb * kBK, m0);
                    if (EPI == kEpiSwiGLU) {
                        ptx::tma_load_2d(sb, &tmB, full_bar(stage), kb * kBK, n0);
                        ptx::tma_load_2d(sb + 128 * kBK, &tmB2, full_bar(stage), kb * kBK, n0);
                    } else {
                        ptx::tma_load_2d(sb, &tmB, full_bar(stage), kb * kBK, n0);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) __nanosleep(200000);   // let copies already in flight land before tear-down
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::umma_idesc(0 /*E4M3*/, 0 /*E4M3*/, kBM, kBN);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            int t = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
                const int buf = t & 1;
                if (!ptx::mbar_wait(tempty_bar(buf), ((t >> 1) & 1u) ^ 1u, p.status, 2)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * kBN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, p.status, 3)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t sa = smem_base + stage * kStageBytes, sb = sa + kABytes;
                    const uint64_t da = ptx::smem_desc_sw128_kmajor(sa), db = ptx::smem_desc_sw128_kmajor(sb);
#pragma unroll
                    for (int k = 0; k < kBK / 32; ++k)   // 32 bytes of K per instruction: +2 in 16-byte units
                        ptx::umma_f8f6f4(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0);
                    ptx::umma_commit(empty_bar(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit(tfull_bar(buf));
            }
            if (!ok) __nanosleep(200000);
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;                         // TMEM lane quadrant this warp may read
        OutT* Cbase = static_cast<OutT*>(p.C);
        const bool ld_ok = ((p.ldc * (long long)sizeof(OutT)) % 16 == 0) && aligned16(p.C);
        int t = 0; bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
            const int buf = t & 1;
            int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            const int row = tm * kBM + q * 32 + lane;
            const int n0 = tn * kOutCols;
            if (!ptx::mbar_wait(tfull_bar(buf), (t >> 1) & 1u, p.status, 4)) { ok = false; break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kBN;
            float rs = 1.0f;
            if (EPI != kEpiTensor) rs = (row < p.M) ? __ldg(p.row_scale + row) : 0.0f;
#pragma unroll 1
            for (int c = 0; c < kOutCols / 32; ++c) {
                uint32_t r[32];
                float v[32];
                const int col0 = n0 + c * 32;
                ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
                if (EPI == kEpiSwiGLU) {
                    uint32_t ru[32];
                    ptx::tmem_ld_32x32b_x32(taddr + 128 + c * 32, ru);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int col = col0 + i;
                        const float sg = (col < p.N) ? __ldg(p.col_scale + col) : 0.0f;
                        const float su = (col < p.N) ? __ldg(p.col_scale2 + col) : 0.0f;
                        const float g = __uint_as_float(r[i]) * (rs * sg);
                        const float u = __uint_as_float(ru[i]) * (rs * su);
                        v[i] = g / (1.0f + __expf(-g)) * u;
                    }
                } else {
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float s;
                        if (EPI == kEpiTensor) s = p.alpha;
                        else { const int col = col0 + i; s = rs * ((col < p.N) ? __ldg(p.col_scale + col) : 0.0f); }
                        v[i] = __uint_as_float(r[i]) * s;
                    }
                }
                if (row < p.M && col0 < p.N) {
                    const int valid = min(32, p.N - col0);
                    OutPack<OutT>::store32(Cbase + (long long)row * p.ldc + col0, v, ld_ok && valid == 32, valid);
                }
            }
            // accumulator drained: hand the TMEM buffer back to the MMA warp
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty_bar(buf));
        }
    }

    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace fp8
}  // namespace b200q
