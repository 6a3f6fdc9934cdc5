// FP8 E4M3 GEMM for sm_100a:  C[M,N] = epilogue( A[M,K] * B[N,K]^T ), fp32 accumulate.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0    TMA producer  : 128-byte-swizzled A (128 x 128 B) and B (BN x 128 B) tiles into a
//                             shared-memory ring, completion on "full" mbarriers
//   warp 1    MMA issuer    : one elected thread issues tcgen05.mma kind::f8f6f4 (128 x BN x 32)
//                             reading shared memory through matrix descriptors, accumulating into
//                             TMEM; tcgen05.commit releases ring slots and publishes accumulators
//   warps 2-5 epilogue      : tcgen05.ld the 128 x BN fp32 accumulator (one TMEM lane = one row),
//                             apply the scale rule, cast to the output type, 16-byte stores
// TMEM holds two accumulators, so the epilogue of tile i overlaps the main loop of tile i+1.
// No cluster, no multicast loads.
//
// With the all-reduce fused in (the row-parallel down projection of the tensor-parallel MLP) the
// CTA has four more warps, the reducers.  The epilogue writes fp32 partial tiles into this rank's
// symmetric buffer and counts finished tiles per group of tile rows; the warp that completes a
// group raises this rank's flag for it on every rank; the reducers of every CTA wait until all
// ranks have raised a group's flag, then add that group's partials across ranks through the
// NVSwitch (multimem.ld_reduce, or plain peer loads in rank order), round once to bf16 and
// broadcast the result to every rank (multimem.st, or peer stores).  The reduction of group g runs
// under the main loop of group g+1; only the last group's reduction is exposed.  It replaces
// GEMM -> ncclAllReduce of op/nccl/nccl_mlp_test.cu:170-195 by one kernel.
//
// Semantics follow the reference: operands K-contiguous, C = A * B^T (op/cpu/cpu_ops.cpp:95-113);
// per-tensor scales are not MMA operands, the epilogue multiplies the fp32 accumulator
// (op/test/arch_primitives/ptx_mma_fp8.cu:16-23); the output cast is round-to-nearest-even from
// fp32 at the very end (op/test/arch_primitives/ptx_mma_fp4.cu:277-282).
#pragma once
#include "common.cuh"
#include "ptx.cuh"
#include "ar_common.cuh"

namespace b200q {
namespace fp8 {

constexpr int kBM = 128;
constexpr int kBK = 128;           // bytes == elements for FP8: one 128-byte swizzle row
constexpr int kBaseThreads = 192;
constexpr int kReducerThreads = 128;
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxWorld = arc::kMaxWorld;
constexpr int kMaxGroups = 64;     // tile-row groups tracked by the fused all-reduce

template <int BN>
struct Cfg {
    static constexpr int kABytes = kBM * kBK;                 // 16 KiB
    static constexpr int kBBytes = BN * kBK;
    static constexpr int kStageBytes = kABytes + kBBytes;     // multiple of 1024 for BN % 8 == 0
    static constexpr int kStages = (227 * 1024 - 1024 - 256) / kStageBytes > 6 ? 6 : (227 * 1024 - 1024 - 256) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
    static_assert(kStageBytes % 1024 == 0 && BN % 16 == 0 && BN <= 256, "tile shape");
};

enum Epilogue : int {
    kEpiTensor = 0,   // C = acc * alpha                                  (per-tensor scales)
    kEpiRowCol = 1,   // C = acc * (row_scale[m] * col_scale[n])          (per-token x per-channel)
    kEpiSwiGLU = 2,   // B tile = BN/2 gate rows + BN/2 up rows; C[m,n] = silu(g) * u, BN/2 columns per tile
    kEpiInt32 = 3,    // signed 8-bit operands (kind::i8), C(int32) = acc (+ c_in): exact integer GEMM
};

struct Params {
    int M, N, K;                 // N = number of OUTPUT columns
    void* C;
    long long ldc;               // elements
    float alpha;
    const float* row_scale;      // [M]
    const float* col_scale;      // [N]   (gate scales for SwiGLU)
    const float* col_scale2;     // [N]   (up scales for SwiGLU)
    const int32_t* c_in;         // [M, ldc] int32 added to the integer accumulator, or nullptr (kEpiInt32)
    int tiles_m, tiles_n;
    int group;                   // tile rows that walk the N tiles together
    uint32_t* status;
    int tma_store;               // CTA-pair kernels: bf16 results leave through TMA stores (tensor map valid)
    uint32_t* sched;             // CTA-pair kernels: {next tile, pairs done} for dynamic tile scheduling, or nullptr (static)
    // fused all-reduce (AR kernels only)
    const void* const* partial_ptrs;     // device array [world]: every rank's partial buffer (C is this rank's)
    __nv_bfloat16* const* out_ptrs;      // device array [world]: every rank's bf16 output
    uint32_t* const* flag_ptrs;          // device array [world]: every rank's flag buffer
    const void* partial_mc;              // multicast address of the partial buffers, or nullptr
    __nv_bfloat16* out_mc;               // multicast address of the outputs, or nullptr
    uint32_t* counters;                  // local, zeroed before the launch: [kMaxGroups + 1]
    uint32_t flag_offset_words;
    uint32_t epoch;
    int rank, world;
    int reducer_stride;                  // only CTAs with blockIdx % reducer_stride == 0 reduce (1 = all)
};

template <typename OutT> struct OutPack;
template <> struct OutPack<__nv_bfloat16> {
    template <int W>
    static __device__ __forceinline__ void store(__nv_bfloat16* dst, const float (&v)[W], bool vec, int valid)
    {
        if (vec) {
            uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int i = 0; i < W / 8; ++i) {
                uint4 q;
                q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
                q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
                q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
                q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
                d[i] = q;
            }
        } else {
#pragma unroll
            for (int i = 0; i < W; ++i)
                if (i < valid) dst[i] = __float2bfloat16_rn(v[i]);
        }
    }
};
template <> struct OutPack<float> {
    template <int W>
    static __device__ __forceinline__ void store(float* dst, const float (&v)[W], bool vec, int valid)
    {
        if (vec) {
            float4* d = reinterpret_cast<float4*>(dst);
#pragma unroll
            for (int i = 0; i < W / 4; ++i) d[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < W; ++i)
                if (i < valid) dst[i] = v[i];
        }
    }
};

// Tile order: groups of `group` tile rows walk the N tiles together so that the CTAs running at
// the same time share A and B tiles in L2 (and, with the fused all-reduce, so that whole row
// groups of the output finish early).
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group, int& tm, int& tn)
{
    const int per_group = group * tiles_n;
    const int g = tile / per_group;
    const int first = g * group;
    const int rows = min(group, tiles_m - first);
    const int r = tile - g * per_group;
    tm = first + r % rows;
    tn = r / rows;
}

// bar.sync on a named barrier shared by the reducer warps only
__device__ __forceinline__ void reducer_barrier()
{
    ptx::named_barrier_1<kReducerThreads>();
}

// The work of persistent CTA `cta` of `nctas` (the kernels below pass the block index and the grid size or,
// when several ranks are emulated inside one launch, the CTA's index within its rank).  The tensor maps
// are kernel parameters (__grid_constant__), addressed through pointers.
template <int EPI, typename OutT, int BN, bool AR>
__device__ __forceinline__ void gemm_fp8_body(const CUtensorMap* tmA, const CUtensorMap* tmB, const CUtensorMap* tmB2,
                                              const Params& p, const int cta, const int nctas)
{
    using CF = Cfg<BN>;
    constexpr int kStages = CF::kStages;
    constexpr int kStageBytes = CF::kStageBytes;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int s_abort;
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
    constexpr int kOutCols = (EPI == kEpiSwiGLU) ? BN / 2 : BN;   // output columns per tile
    constexpr int kCW = (kOutCols % 32 == 0) ? 32 : 16;           // columns per TMEM load

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull_bar(b), 1); ptx::mbar_init(tempty_bar(b), 4); }
        ptx::fence_mbar_init();
        s_abort = 0;
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
            ptx::tma_prefetch_desc(tmA);
            ptx::tma_prefetch_desc(tmB);
            if (EPI == kEpiSwiGLU) ptx::tma_prefetch_desc(tmB2);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int tile = cta; tile < num_tiles && ok; tile += nctas) {
                int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
                const int m0 = tm * kBM, n0 = tn * kOutCols;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 1)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * kStageBytes, sb = sa + CF::kABytes;
                    ptx::mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
                    ptx::tma_load_2d(sa, tmA, full_bar(stage), kb * kBK, m0);
                    if (EPI == kEpiSwiGLU) {
                        ptx::tma_load_2d(sb, tmB, full_bar(stage), kb * kBK, n0);
                        ptx::tma_load_2d(sb + (BN / 2) * kBK, tmB2, full_bar(stage), kb * kBK, n0);
                    } else {
                        ptx::tma_load_2d(sb, tmB, full_bar(stage), kb * kBK, n0);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) __nanosleep(200000);   // let copies already in flight land before tear-down
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = (EPI == kEpiInt32) ? ptx::umma_idesc_i8(kBM, BN) : ptx::umma_idesc(0 /*E4M3*/, 0 /*E4M3*/, kBM, BN);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            int t = 0;
            for (int tile = cta; tile < num_tiles && ok; tile += nctas, ++t) {
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
                    for (int k = 0; k < kBK / 32; ++k) {  // 32 bytes of K per instruction: +2 in 16-byte units
                        if (EPI == kEpiInt32) ptx::umma_i8(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0);
                        else ptx::umma_f8f6f4(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0);
                    }
                    ptx::umma_commit(empty_bar(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::umma_commit(tfull_bar(buf));
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;                         // TMEM lane quadrant this warp may read
        OutT* Cbase = static_cast<OutT*>(p.C);
        const bool ld_ok = ((p.ldc * (long long)sizeof(OutT)) % 16 == 0) && aligned16(p.C);
        int t = 0; bool ok = true;
        for (int tile = cta; tile < num_tiles && ok; tile += nctas, ++t) {
            const int buf = t & 1;
            int tm, tn; tile_coords(tile, p.tiles_m, p.tiles_n, p.group, tm, tn);
            const int row = tm * kBM + q * 32 + lane;
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
                if (row < p.M && col0 < p.N) {
                    const int valid = min(kCW, p.N - col0);
                    OutPack<OutT>::template store<kCW>(Cbase + (long long)row * p.ldc + col0, v, ld_ok && valid == kCW, valid);
                }
            }
            // accumulator drained: hand the TMEM buffer back to the MMA warp
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty_bar(buf));
            if (AR) {
                // this warp's share of the tile is in memory: count it; the warp that completes
                // the group tells every rank
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    const int g = tm / p.group;
                    const uint32_t target = 4u * min(p.group, p.tiles_m - g * p.group) * p.tiles_n;
                    if (atomicAdd(p.counters + g, 1u) + 1u == target) {
                        __threadfence_system();
                        for (int r = 0; r < p.world; ++r)
                            arc::st_release_sys(p.flag_ptrs[r] + p.flag_offset_words + g * kMaxWorld + p.rank, p.epoch);
                    }
                }
            }
        }
    } else if (AR) {
        // ---------------------------------------------------------------- reducers
        const int rt = threadIdx.x - kBaseThreads;
        const int groups = (p.tiles_m + p.group - 1) / p.group;
        const uint32_t* my_flags = p.flag_ptrs[p.rank] + p.flag_offset_words;
        bool ok = true;
        for (int g = 0; g < groups && ok; ++g) {
            if (rt < p.world && !arc::wait_flag(my_flags + g * kMaxWorld + rt, p.epoch, p.status, 5)) s_abort = 1;
            reducer_barrier();
            if (*reinterpret_cast<volatile int*>(&s_abort)) { ok = false; break; }
            const long long row0 = static_cast<long long>(g) * p.group * kBM;
            const long long rows = min(static_cast<long long>(p.group) * kBM, static_cast<long long>(p.M) - row0);
            const long long vecs = rows * p.N / 8;                  // 8 fp32 -> 8 bf16 (16 bytes)
            const long long v0 = vecs * p.rank / p.world, v1 = vecs * (p.rank + 1) / p.world;
            const long long base = row0 * p.N;
            // kUnroll independent 32-byte reductions in flight per thread: the round trip through the
            // switch is microseconds, so throughput comes from the number of loads outstanding
            constexpr int kUnroll = 8;
            const int rstride = p.reducer_stride;
            const long long nred = (nctas + rstride - 1) / rstride;       // CTAs that take part
            const long long stride = nred * kReducerThreads;
            if (cta % rstride != 0) continue;
            for (long long vb = v0 + (cta / rstride) * static_cast<long long>(kReducerThreads) + rt; vb < v1;
                 vb += stride * kUnroll) {
                uint4 o[kUnroll];
                long long e[kUnroll];
                bool valid[kUnroll];
                constexpr bool kBf = sizeof(OutT) == 2;          // partial tiles are stored as OutT
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) { valid[u] = vb + u * stride < v1; e[u] = base + (vb + u * stride) * 8; }
                if (p.partial_mc != nullptr) arc::reduce8xU<true, kBf, kUnroll>(p.partial_ptrs, p.partial_mc, p.world, e, valid, o);
                else arc::reduce8xU<false, kBf, kUnroll>(p.partial_ptrs, p.partial_mc, p.world, e, valid, o);
#pragma unroll
                for (int u = 0; u < kUnroll; ++u)
                    if (valid[u]) {
                        if (p.out_mc != nullptr) arc::broadcast8<true>(p.out_ptrs, p.out_mc, p.world, e[u], o[u]);
                        else arc::broadcast8<false>(p.out_ptrs, p.out_mc, p.world, e[u], o[u]);
                    }
            }
        }
        // every rank's broadcasts into this rank's output must have landed before the kernel ends
        reducer_barrier();
        if (ok) {
            if (rt == 0) {
                __threadfence_system();
                if (atomicAdd(p.counters + kMaxGroups, 1u) + 1u == static_cast<uint32_t>(nctas))
                    for (int r = 0; r < p.world; ++r)
                        arc::st_release_sys(p.flag_ptrs[r] + p.flag_offset_words + kMaxGroups * kMaxWorld + p.rank, p.epoch);
            }
            if (rt < p.world) arc::wait_flag(my_flags + kMaxGroups * kMaxWorld + rt, p.epoch, p.status, 6);
        }
    }

    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int EPI, typename OutT, int BN, bool AR>
__global__ void __launch_bounds__(kBaseThreads + (AR ? kReducerThreads : 0), 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmB2, const Params p)
{
    gemm_fp8_body<EPI, OutT, BN, AR>(&tmA, &tmB, &tmB2, p, blockIdx.x, gridDim.x);
}

// The down projection with the fused all-reduce for every rank of a small world inside ONE launch on ONE
// device: CTAs [r * ctas_per_rank, (r + 1) * ctas_per_rank) play rank r on that rank's operands and buffers
// (all in this device's memory).  Launched cooperatively, so the CTAs of all "ranks" are resident together
// and the flags they raise for one another are seen; separate launches that wait on one another on one
// device would have no such guarantee.  Peer loads/stores only.
constexpr int kOneDeviceMaxWorld = 4;
struct OneDeviceArgs {
    alignas(64) CUtensorMap tmA[kOneDeviceMaxWorld];
    alignas(64) CUtensorMap tmB[kOneDeviceMaxWorld];
    Params p[kOneDeviceMaxWorld];
    int ctas_per_rank;
};
template <typename OutT>
__global__ void __launch_bounds__(kBaseThreads + kReducerThreads, 1)
gemm_fp8_allreduce_one_device_kernel(const __grid_constant__ OneDeviceArgs a)
{
    const int r = blockIdx.x / a.ctas_per_rank;
    gemm_fp8_body<kEpiRowCol, OutT, 256, true>(&a.tmA[r], &a.tmB[r], &a.tmB[r], a.p[r], blockIdx.x % a.ctas_per_rank,
                                               a.ctas_per_rank);
}

}  // namespace fp8
}  // namespace b200q
