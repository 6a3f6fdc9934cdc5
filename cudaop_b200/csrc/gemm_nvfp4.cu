// NVFP4 block-scaled GEMM for sm_100a:
//   C[M,N] (bf16) = ( (A .* sfa) * (B .* sfb)^T ) * (global_a * global_b)
// A[M,K], B[N,K]: E2M1, two per byte, low nibble = lower K (op/test/arch_primitives/ptx_mma_fp4.cu:120-130);
// one UE4M3 scale per 16 consecutive K (ptx_mma_fp4.cu:55-65, decoders :285-309); fp32 accumulate, one
// round-to-nearest-even cast at the end (:277-282).  The global scales are ordinary per-tensor
// scales: they multiply the accumulator in the epilogue.
//
// Kernel: the FP8 kernel's structure (persistent CTA, TMA producer warp / MMA issuer warp / four
// epilogue warps, 128-byte-swizzled operand ring) with tcgen05.mma kind::mxf4nvf4.block_scale
// (128 x BN x 64 per instruction, scale_vec::4X = four scales per row per instruction).  The tensor
// core reads the scales from TMEM, laid out as "row r -> lane r % 32, column r / 32, byte = scale
// index", so the scales travel in 512-byte blocks (128 rows x 4 scales, byte offset
// (r % 32) * 16 + (r / 32) * 4 + j): b200q_nvfp4_swizzle_sf writes that layout, plain bulk copies
// bring the blocks of a K-slab into shared memory with the operands, and the issuing thread moves
// each block into TMEM with tcgen05.cp (32x128b.warpx4) right before the MMAs that use it — the
// tensor pipe executes its operations in issue order, so no wait sits between copy and MMA.
// TMEM: two BN-column accumulators when they fit next to the scale columns (BN <= 192), else one.
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

#include <cstdio>
#include <mutex>

namespace b200q {
namespace nvfp4 {

using ptx::bulk_load;

constexpr int kBM = 128;
constexpr int kBKBytes = 128;            // 256 E2M1 elements per row and stage
constexpr int kBKElems = 256;
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kSfBlockBytes = 512;       // 128 rows x 4 scales
constexpr uint32_t kTmemCols = 512;

template <int BN>
struct Cfg {
    // scale row-blocks (of 128 rows) a B tile can span: tiles start at multiples of BN, so at offset
    // 0 or 64 inside their first block.  BN must be a multiple of 64: the tensor core takes the B
    // scales from a TMEM address that is a multiple of two columns (64 rows of B); a 224-wide tile,
    // whose odd tiles start 32 or 96 rows into a block, raised "misaligned address".
    static_assert(BN % 64 == 0, "B tile width must be a multiple of 64 for the scale-factor address");
    static constexpr int kMaxOff = (BN % 128 == 0) ? 0 : 64;
    static constexpr int kNB = (kMaxOff + BN + 127) / 128;
    static constexpr int kABytes = kBM * kBKBytes;                  // 16 KiB
    static constexpr int kBBytes = BN * kBKBytes;
    static constexpr int kSfaBytes = 4 * kSfBlockBytes;             // 4 K-steps
    static constexpr int kSfbBytes = kNB * 4 * kSfBlockBytes;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // multiple of 1024
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
    static constexpr int kAccBufs = (2 * BN + 16 + 16 * kNB <= 512) ? 2 : 1;   // two accumulators when they fit beside the scales
    static constexpr int kSfaCol = kAccBufs * BN;                   // first scale column in TMEM
    static constexpr int kSfbCol = kSfaCol + 16;
    static_assert(kSfbCol + 4 * 4 * kNB <= 512, "TMEM budget");
    static_assert(kStageBytes % 1024 == 0, "stage alignment");
};

struct Params {
    int M, N, K;
    __nv_bfloat16* C;
    float alpha;
    const uint8_t* sfa;      // swizzled: [ceil(M/128)][K/64] blocks of 512 bytes
    const uint8_t* sfb;      // swizzled: [ceil(N/128)][K/64]
    int tiles_m, tiles_n;
    uint32_t* status;
};

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

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p)
{
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + kStages * C::kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - ptx::smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (p.K + kBKElems - 1) / kBKElems;
    const int k64_total = p.K / 64;                      // scale blocks along K
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int sf_rows_b = (p.N + 127) / 128;

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
        // ------------------------------------------------------------ producer
        if (ptx::elect_one()) {
            ptx::tma_prefetch_desc(&tmA);
            ptx::tma_prefetch_desc(&tmB);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                const int m0 = tm * kBM, n0 = tn * BN;
                const int rb0 = n0 / 128;                 // first scale row-block of this B tile
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 1)) { ok = false; break; }
                    const int ksteps = min(4, k64_total - 4 * kb);            // 64-element steps in this slab
                    const uint32_t sf_bytes = ksteps * kSfBlockBytes;
                    int nb = 0;
                    for (int i = 0; i < C::kNB; ++i) nb += (rb0 + i) < sf_rows_b;
                    const uint32_t sa = smem_base + stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes, ssfa = sb + C::kBBytes, ssfb = ssfa + C::kSfaBytes;
                    ptx::mbar_arrive_expect_tx(full_bar(stage), C::kABytes + C::kBBytes + sf_bytes * (1 + nb));
                    ptx::tma_load_2d(sa, &tmA, full_bar(stage), kb * kBKBytes, m0);
                    ptx::tma_load_2d(sb, &tmB, full_bar(stage), kb * kBKBytes, n0);
                    bulk_load(ssfa, p.sfa + (static_cast<size_t>(tm) * k64_total + 4 * kb) * kSfBlockBytes, sf_bytes,
                              full_bar(stage));
                    for (int i = 0; i < C::kNB; ++i)
                        if (rb0 + i < sf_rows_b)
                            bulk_load(ssfb + i * 4 * kSfBlockBytes,
                                      p.sfb + (static_cast<size_t>(rb0 + i) * k64_total + 4 * kb) * kSfBlockBytes,
                                      sf_bytes, full_bar(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (ptx::elect_one()) {
            // E2M1 operands (format code 1 for the 4-bit kinds), UE4M3 scales (0), scale ids 0: with
            // four scales per instruction every byte of the 32-bit scale column is used
            constexpr uint32_t idesc = ptx::umma_idesc_block_scaled(1, 1, kBM, BN, 0, 0, 0);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            int t = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
                const int buf = (C::kAccBufs == 2) ? (t & 1) : 0;
                const uint32_t par = (C::kAccBufs == 2) ? ((t >> 1) & 1u) : (t & 1u);
                if (!ptx::mbar_wait(tempty_bar(buf), par ^ 1u, p.status, 2)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                const uint32_t sfb_col_off = ((tn * BN) % 128) / 32;      // tile start inside its first scale block
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(full_bar(stage), phase, p.status, 3)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const int ksteps = min(4, k64_total - 4 * kb);
                    const uint32_t sa = smem_base + stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes, ssfa = sb + C::kBBytes, ssfb = ssfa + C::kSfaBytes;
                    const uint64_t da = ptx::smem_desc_sw128_kmajor(sa), db = ptx::smem_desc_sw128_kmajor(sb);
                    // descriptors advance in 16-byte units: one 512-byte scale block = 32
                    const uint64_t dsfa = ptx::smem_desc_noswizzle_kmajor(ssfa, 16, 128), dsfb = ptx::smem_desc_noswizzle_kmajor(ssfb, 16, 128);
                    const uint32_t tsfa = tmem_base + C::kSfaCol, tsfb = tmem_base + C::kSfbCol;
                    auto kstep = [&](int ks) {
                        // scales of this K-step: one 512-byte block for A, kNB blocks for B
                        ptx::tmem_cp_32x128b_warpx4(tsfa + 4 * ks, dsfa + 32u * ks);
#pragma unroll
                        for (int i = 0; i < C::kNB; ++i)
                            ptx::tmem_cp_32x128b_warpx4(tsfb + 4 * C::kNB * ks + 4 * i, dsfb + 32u * (i * 4 + ks));
                        ptx::umma_mxf4nvf4(d_tmem, da + 2u * ks, db + 2u * ks, idesc, tsfa + 4 * ks,
                                           tsfb + 4 * C::kNB * ks + sfb_col_off, (kb | ks) != 0);
                    };
                    if (ksteps == 4) {             // the single issuing thread is on the critical path: no loop overhead
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) kstep(ks);
                    } else {
                        for (int ks = 0; ks < ksteps; ++ks) kstep(ks);
                    }
                    ptx::umma_commit(empty_bar(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit(tfull_bar(buf));
            }
            if (!ok) __nanosleep(200000);
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;
        const bool vec_ok = ((static_cast<long long>(p.N) * 2) % 16 == 0) && aligned16(p.C);
        int t = 0; bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
            const int buf = (C::kAccBufs == 2) ? (t & 1) : 0;
            const uint32_t par = (C::kAccBufs == 2) ? ((t >> 1) & 1u) : (t & 1u);
            int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            const int row = tm * kBM + q * 32 + lane;
            const int n0 = tn * BN;
            if (!ptx::mbar_wait(tfull_bar(buf), par, p.status, 4)) { ok = false; break; }
            ptx::tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
                ptx::tmem_ld_wait();
                const int col0 = n0 + c * 32;
                if (row < p.M && col0 < p.N) {
                    __nv_bfloat16* dst = p.C + static_cast<size_t>(row) * p.N + col0;
                    const int valid = min(32, p.N - col0);
                    if (vec_ok && valid == 32) {
                        uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * p.alpha, __uint_as_float(r[8 * i + 1]) * p.alpha);
                            o.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * p.alpha, __uint_as_float(r[8 * i + 3]) * p.alpha);
                            o.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * p.alpha, __uint_as_float(r[8 * i + 5]) * p.alpha);
                            o.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * p.alpha, __uint_as_float(r[8 * i + 7]) * p.alpha);
                            d[i] = o;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]) * p.alpha);
                    }
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
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Row-major scales [rows, K/16] -> blocked layout [ceil(rows/128)][K/64][512 bytes]; rows beyond
// `rows` are written as zero scales.  One thread per output 32-bit word (four scales of one row).
__global__ void swizzle_sf_kernel(const uint8_t* __restrict__ src, uint32_t* __restrict__ dst, int rows, int k64)
{
    const size_t total = static_cast<size_t>((rows + 127) / 128) * k64 * 128;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int w = static_cast<int>(i % 128);          // word inside the block: (r % 32) * 4 + (r / 32)
        const size_t blk = i / 128;
        const int kb = static_cast<int>(blk % k64);
        const int rb = static_cast<int>(blk / k64);
        const int r = rb * 128 + (w >> 2) + 32 * (w & 3);
        uint32_t v = 0;
        if (r < rows) v = *reinterpret_cast<const uint32_t*>(src + (static_cast<size_t>(r) * k64 + kb) * 4);
        dst[i] = v;
    }
}

template <int BN>
cudaError_t launch(const CUtensorMap& tmA, const CUtensorMap& tmB, Params p, cudaStream_t stream)
{
    auto kernel = gemm_nvfp4_kernel<BN>;
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
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int tiles = p.tiles_m * p.tiles_n;
    kernel<<<tiles < sms ? tiles : sms, kThreads, Cfg<BN>::kSmemBytes, stream>>>(tmA, tmB, p);
    return cudaGetLastError();
}

int g_tile_n = 256;     // B tile width: 128, 192 or 256 (b200q_nvfp4_set_tile_n)
int g_use_2cta = 1;     // 1 (default): CTA-pair kernel (gemm_nvfp4_2cta.cu) for tile widths 192 / 256 (b200q_nvfp4_set_2cta)

}  // namespace nvfp4
}  // namespace b200q

namespace b200q {
// gemm_nvfp4_2cta.cu: the CTA-pair kernel (256-row tiles, bn = 192 or 256 columns)
int gemm_nvfp4_blocked_pair(const void* Aq, const void* SFA_blocked, const void* Bq, const void* SFB_blocked, void* C, int M, int N,
                            int K, float global_a, float global_b, int bn, void* stream);
}

extern "C" {

size_t b200q_nvfp4_sf_bytes(int rows, int K)
{
    if (rows <= 0 || K <= 0 || K % 64 != 0) return 0;
    return static_cast<size_t>((rows + 127) / 128) * (K / 64) * 512;
}

int b200q_nvfp4_swizzle_sf(const void* sf_rowmajor, void* sf_blocked, int rows, int K, void* stream)
{
    using namespace b200q;
    if (sf_rowmajor == nullptr || sf_blocked == nullptr || rows <= 0 || K <= 0 || K % 64 != 0)
        return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(sf_rowmajor) & 3u) || !aligned16(sf_blocked)) return cudaErrorInvalidValue;
    const size_t words = b200q_nvfp4_sf_bytes(rows, K) / 4;
    const int grid = static_cast<int>((words + 255) / 256 < 4096 ? (words + 255) / 256 : 4096);
    nvfp4::swizzle_sf_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(sf_rowmajor), static_cast<uint32_t*>(sf_blocked), rows, K / 64);
    return cudaGetLastError();
}

int b200q_nvfp4_set_tile_n(int bn)
{
    if (bn != 128 && bn != 192 && bn != 256) return cudaErrorInvalidValue;
    b200q::nvfp4::g_tile_n = bn;
    return 0;
}

int b200q_nvfp4_set_2cta(int on)
{
    b200q::nvfp4::g_use_2cta = on ? 1 : 0;
    return 0;
}

int b200q_gemm_nvfp4_blocked(const void* Aq, const void* SFA_blocked, const void* Bq, const void* SFB_blocked, void* C,
                             int M, int N, int K, float global_a, float global_b, void* stream)
{
    using namespace b200q;
    if (Aq == nullptr || SFA_blocked == nullptr || Bq == nullptr || SFB_blocked == nullptr || C == nullptr)
        return cudaErrorInvalidValue;
    if (M <= 0 || N <= 0 || K <= 0 || K % 64 != 0) return cudaErrorInvalidValue;
    if (!aligned16(Aq) || !aligned16(Bq) || !aligned16(SFA_blocked) || !aligned16(SFB_blocked))
        return cudaErrorInvalidValue;
    nvfp4::Params p{};
    p.M = M; p.N = N; p.K = K; p.C = static_cast<__nv_bfloat16*>(C); p.alpha = global_a * global_b;
    p.sfa = static_cast<const uint8_t*>(SFA_blocked); p.sfb = static_cast<const uint8_t*>(SFB_blocked);
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    const int bn = nvfp4::g_tile_n;
    if (nvfp4::g_use_2cta && bn != 128 && M > 128)
        return gemm_nvfp4_blocked_pair(Aq, SFA_blocked, Bq, SFB_blocked, C, M, N, K, global_a, global_b, bn, stream);
    CUtensorMap tmA, tmB;
    if (!make_tmap_2d_u8(&tmA, Aq, M, K / 2, K / 2, nvfp4::kBM, nvfp4::kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    if (!make_tmap_2d_u8(&tmB, Bq, N, K / 2, K / 2, bn, nvfp4::kBKBytes, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (bn == 128) return nvfp4::launch<128>(tmA, tmB, p, s);
    if (bn == 256) return nvfp4::launch<256>(tmA, tmB, p, s);
    return nvfp4::launch<192>(tmA, tmB, p, s);
}

size_t b200q_gemm_nvfp4_workspace_bytes(int M, int N, int K)
{
    const size_t a = b200q_nvfp4_sf_bytes(M, K), b = b200q_nvfp4_sf_bytes(N, K);
    return (a == 0 || b == 0) ? 0 : a + b;
}

int b200q_gemm_nvfp4(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C, int M, int N, int K,
                     float global_a, float global_b, void* workspace, void* stream)
{
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15u)) return cudaErrorInvalidValue;
    const size_t a_bytes = b200q_nvfp4_sf_bytes(M, K);
    if (a_bytes == 0) return cudaErrorInvalidValue;
    uint8_t* wa = static_cast<uint8_t*>(workspace);
    uint8_t* wb = wa + a_bytes;
    int e = b200q_nvfp4_swizzle_sf(SFA, wa, M, K, stream);
    if (e != 0) return e;
    e = b200q_nvfp4_swizzle_sf(SFB, wb, N, K, stream);
    if (e != 0) return e;
    return b200q_gemm_nvfp4_blocked(Aq, wa, Bq, wb, C, M, N, K, global_a, global_b, stream);
}

// ------------------------------------------------------------------------------------------
// b200q_gemm_nvfp4_static: the row-major-scales GEMM for callers that cannot hand in a workspace.
//
// Some hosts of this library have no way to obtain device memory at the moment of the call: an
// inference server that reserved the whole GPU for its own pool at start-up (a cudaMalloc from a
// plug-in then fails, or fragments the pool's view of the device), a real-time loop that must not
// hit the allocator's device-wide synchronisation, or code running where the only memory it owns
// is the operands it was given.  For them the blocked copies of the two scale arrays live in a
// fixed array that is part of the library image, kStaticScratchBytes per GPU that loads the
// library, held until the process exits.
//
//   * First call on a device: the entry point looks up the array's device address
//     (cudaGetSymbolAddress on the symbol below; in host code the symbol's name is only a handle,
//     never an address a kernel may be given) and caches it for that device.  Make that first
//     call outside any stream capture.
//   * Limit: b200q_gemm_nvfp4_workspace_bytes(M, N, K) <= kStaticScratchBytes (8 MiB: up to
//     M = N = K = 8192); larger problems are refused with cudaErrorInvalidValue and a message on
//     stderr.  Use b200q_gemm_nvfp4 with your own workspace for those.
//   * One array per device, shared by every call: two calls whose kernels can overlap on the GPU
//     (different streams, or graphs replayed concurrently) would overwrite each other's scales.
//     Calls on one stream are safe.  Nothing in the array has to be zero beforehand: the
//     rewrite kernel writes every byte it later reads, zero padding of ragged row blocks included,
//     so whatever an earlier call left behind is never observed.
//   * No allocation of any kind happens here: no cudaMalloc / cudaFree, no library call that
//     allocates.

namespace b200q {
namespace nvfp4 {

constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) uint8_t g_static_sf_scratch[kStaticScratchBytes];

namespace {
std::mutex g_static_mu;
uint8_t* g_static_ptr[64] = {};        // device address of g_static_sf_scratch, per device ordinal
}  // namespace

// Device address of the scratch array on the current device, looked up once per device.
static cudaError_t static_scratch(uint8_t** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_sf_scratch);      // this device is current: its copy of the symbol
        if (e != cudaSuccess) return e;
        if (p == nullptr) return cudaErrorInvalidSymbol;
        g_static_ptr[dev] = static_cast<uint8_t*>(p);
    }
    *out = g_static_ptr[dev];
    return cudaSuccess;
}

}  // namespace nvfp4
}  // namespace b200q

size_t b200q_gemm_nvfp4_static_max_bytes(void) { return b200q::nvfp4::kStaticScratchBytes; }

int b200q_gemm_nvfp4_static(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C, int M, int N, int K,
                            float global_a, float global_b, void* stream)
{
    const size_t need = b200q_gemm_nvfp4_workspace_bytes(M, N, K);
    if (need == 0) return cudaErrorInvalidValue;                 // bad sizes (K % 64, non-positive)
    if (need > b200q::nvfp4::kStaticScratchBytes) {
        std::fprintf(stderr,
                     "b200q_gemm_nvfp4_static: M=%d N=%d K=%d needs %zu bytes of scale scratch, the built-in array holds %zu; "
                     "use b200q_gemm_nvfp4 with a caller-owned workspace\n",
                     M, N, K, need, b200q::nvfp4::kStaticScratchBytes);
        return cudaErrorInvalidValue;
    }
    uint8_t* scratch = nullptr;
    const cudaError_t e = b200q::nvfp4::static_scratch(&scratch);
    if (e != cudaSuccess) return e;
    return b200q_gemm_nvfp4(Aq, SFA, Bq, SFB, C, M, N, K, global_a, global_b, scratch, stream);
}

}  // extern "C"
