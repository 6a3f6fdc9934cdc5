// Grouped (ragged-M) FP8 GEMM for sm_100a: the quantized counterpart of the reference's grouped GEMM
//   gmm(a, b, batch_sizes, trans_b)   (op/grouped_gemm/cudaop_grouped_gemm/ops.py:76-83,
//   dispatch op/grouped_gemm/csrc/grouped_gemm.cuh:96-328; consumer op/lora_moe/gmm_ops.py:7-15)
// The rows of A[tokens, K] are split into E consecutive groups of batch_sizes[e] rows; group e is multiplied by
// its own weight matrix B[e][N, K] (K contiguous, the reference's trans_b = True layout):
//   C[t, n] (bf16) = (sum_k A[t, k] * B[e(t)][n, k]) * a_scale[t] * b_scale[e(t)][n]
// A, B hold E4M3 bytes; a_scale is one fp32 per token, b_scale one fp32 per expert and output channel.
//
// One persistent launch for all groups (the reference builds per-group problem descriptors for a CUTLASS grouped
// kernel; here every CTA derives its tiles from batch_sizes itself): each CTA reads batch_sizes into shared
// memory, builds the prefix sums of rows and of 128-row tiles, and walks tile numbers cta, cta + grid, ...;
// a tile number maps to (group, row tile inside the group, column tile) by a search in the prefix array.
// A is ONE tensor map over all tokens: a row tile that reaches past its group's last row simply carries rows of
// the next group, which the epilogue does not store.  B is one tensor map over [E * N, K]; a column tile that
// reaches past N carries rows of the next expert, whose columns are not stored either.
// Pipeline as in gemm_fp8.cuh: warp 0 TMA producer, warp 1 tcgen05.mma (kind::f8f6f4, 128 x 256 x 32) into two
// TMEM accumulators, warps 2-5 epilogue (scale, cast, 16-byte stores).  No cluster, no multicast.
#include "gemm_fp8.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace gmm {

using fp8::kBK;
using fp8::kBM;
constexpr int kBN = 256;
constexpr int kThreads = 192;
constexpr int kMaxGroups = 1024;
using CF = fp8::Cfg<kBN>;
// after the operand ring and the barriers: row prefix [E + 1] and tile prefix [E + 1]
constexpr int kSmemBytes = CF::kSmemBytes + 2 * (kMaxGroups + 1) * 4;

struct Params {
    int tokens, N, K, E;
    const long long* batch_sizes;      // [E] rows per group (device memory)
    __nv_bfloat16* C;                  // [tokens, N]
    const float* a_scale;              // [tokens]
    const float* b_scale;              // [E, N]
    int tiles_n;
    uint32_t* status;
};

// group of row-tile number rt: the last e with tile_start[e] <= rt
__device__ __forceinline__ int find_group(const int* tile_start, int E, int rt)
{
    int lo = 0, hi = E - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tile_start[mid] <= rt) lo = mid; else hi = mid - 1;
    }
    return lo;
}

__global__ void __launch_bounds__(kThreads, 1)
gmm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p)
{
    constexpr int kStages = CF::kStages;
    constexpr int kStageBytes = CF::kStageBytes;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kStages * kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
    int* row_start = reinterpret_cast<int*>(smem_gen + (bar_base - smem_base) + 256);      // [E + 1]
    int* tile_start = row_start + (kMaxGroups + 1);                                        // [E + 1]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), 4); }
        ptx::fence_mbar_init();
        // prefix sums over the groups (E is small: one thread); rows beyond `tokens` are cut off
        int rows = 0, tiles = 0;
        for (int e = 0; e < p.E; ++e) {
            row_start[e] = rows; tile_start[e] = tiles;
            long long bs = p.batch_sizes[e];
            if (bs < 0) bs = 0;
            if (bs > p.tokens - rows) bs = p.tokens - rows;
            rows += static_cast<int>(bs);
            tiles += (static_cast<int>(bs) + kBM - 1) / kBM;
        }
        row_start[p.E] = rows; tile_start[p.E] = tiles;
    }
    if (warp == 1) { ptx::tmem_alloc(tmem_slot, fp8::kTmemCols); ptx::tmem_relinquish(); }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const int num_tiles = tile_start[p.E] * p.tiles_n;

    // tile number -> group e, first row m0, one past the group's last row, first output column
    auto tile_info = [&](int tile, int& e, int& m0, int& m_end, int& n0) {
        const int rt = tile / p.tiles_n;
        e = find_group(tile_start, p.E, rt);
        m0 = row_start[e] + (rt - tile_start[e]) * kBM;
        m_end = row_start[e + 1];
        n0 = (tile - rt * p.tiles_n) * kBN;
    };

    if (warp == 0) {
        if (ptx::elect_one()) {
            ptx::tma_prefetch_desc(&tmA);
            ptx::tma_prefetch_desc(&tmB);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int e, m0, m_end, n0; tile_info(tile, e, m0, m_end, n0);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * kStageBytes, sb = sa + CF::kABytes;
                    ptx::mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
                    ptx::tma_load_2d(sa, &tmA, full_bar(stage), kb * kBK, m0);
                    ptx::tma_load_2d(sb, &tmB, full_bar(stage), kb * kBK, e * p.N + n0);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp == 1) {
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::umma_idesc(0, 0, kBM, kBN);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            int t = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
                const int buf = t & 1;
                if (!ptx::mbar_wait(tempty_bar(buf), ((t >> 1) & 1u) ^ 1u, p.status, 2)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * 256;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, p.status, 3)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t sa = smem_base + stage * kStageBytes, sb = sa + CF::kABytes;
                    const uint64_t da = ptx::smem_desc_sw128_kmajor(sa), db = ptx::smem_desc_sw128_kmajor(sb);
#pragma unroll
                    for (int k = 0; k < kBK / 32; ++k) ptx::umma_f8f6f4(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0);
                    ptx::umma_commit(empty_bar(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit(tfull_bar(buf));
            }
            if (!ok) __nanosleep(200000);
        }
    } else {
        const int q = warp & 3;
        const bool vec_ok = (p.N % 8 == 0) && aligned16(p.C);
        int t = 0; bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
            const int buf = t & 1;
            int e, m0, m_end, n0; tile_info(tile, e, m0, m_end, n0);
            const int row = m0 + q * 32 + lane;
            if (!ptx::mbar_wait(tfull_bar(buf), (t >> 1) & 1u, p.status, 4)) { ok = false; break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * 256;
            const bool row_ok = row < m_end;                       // rows past the group's end belong to the next group
            const float rs = row_ok ? __ldg(p.a_scale + row) : 0.0f;
            const float* cs = p.b_scale + static_cast<size_t>(e) * p.N;
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c) {
                uint32_t r[32];
                float v[32];
                const int col0 = n0 + c * 32;
                ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int col = col0 + i;
                    v[i] = __uint_as_float(r[i]) * (rs * ((col < p.N) ? __ldg(cs + col) : 0.0f));
                }
                if (row_ok && col0 < p.N) {
                    const int valid = min(32, p.N - col0);
                    fp8::OutPack<__nv_bfloat16>::store<32>(p.C + static_cast<size_t>(row) * p.N + col0, v, vec_ok && valid == 32, valid);
                }
            }
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty_bar(buf));
        }
    }

    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, fp8::kTmemCols);
    }
}

}  // namespace gmm
}  // namespace b200q

extern "C" int b200q_gmm_fp8(const void* A, const float* a_scale, const void* B, const float* b_scale,
                             const long long* batch_sizes_dev, void* C, int tokens, int N, int K, int E, void* stream)
{
    using namespace b200q;
    if (A == nullptr || a_scale == nullptr || B == nullptr || b_scale == nullptr || batch_sizes_dev == nullptr || C == nullptr)
        return cudaErrorInvalidValue;
    if (tokens <= 0 || N <= 0 || K <= 0 || E <= 0 || E > gmm::kMaxGroups || K % 16 != 0) return cudaErrorInvalidValue;
    if (!aligned16(A) || !aligned16(B) || (reinterpret_cast<uintptr_t>(batch_sizes_dev) & 7u)) return cudaErrorInvalidValue;
    if (static_cast<long long>(E) * N > 0x7FFFFFFFLL) return cudaErrorInvalidValue;
    gmm::Params p{};
    p.tokens = tokens; p.N = N; p.K = K; p.E = E; p.batch_sizes = batch_sizes_dev;
    p.C = static_cast<__nv_bfloat16*>(C); p.a_scale = a_scale; p.b_scale = b_scale;
    p.tiles_n = (N + gmm::kBN - 1) / gmm::kBN;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    CUtensorMap tmA, tmB;
    if (!make_tmap_2d_u8(&tmA, A, tokens, K, K, gmm::kBM, gmm::kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    if (!make_tmap_2d_u8(&tmB, B, static_cast<uint64_t>(E) * N, K, K, gmm::kBN, gmm::kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(gmm::gmm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gmm::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    // the tile count depends on batch_sizes, which the host does not read: at most ceil(tokens / 128) + E row tiles
    const long long max_tiles = (static_cast<long long>((tokens + gmm::kBM - 1) / gmm::kBM) + E) * p.tiles_n;
    const int grid = static_cast<int>(max_tiles < sms ? max_tiles : sms);
    gmm::gmm_fp8_kernel<<<grid, gmm::kThreads, gmm::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
    return cudaGetLastError();
}
