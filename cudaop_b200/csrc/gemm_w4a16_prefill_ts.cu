// INT4 weight-only GEMM for prefill shapes with the WEIGHTS as the tensor-memory operand, sm_100a.
//   Y[M,N] (bf16) = X[M,K] (bf16) * dequant(Wq)[N,K]^T,   w[n,k] = q[n,k] * S[n, k/128]
// Wq: two signed nibbles per byte along K, low nibble = lower K
// (op/test/arch_primitives/ptx_mma_integer.cu:93-108); S fp16, one per 128 K, no zero point.
//
// The product is computed transposed, D[n, m] = sum_k q[n,k] x[m,k], so that the operand that has to be
// manufactured (integer weights as bf16) is the MMA's A operand and can live in tensor memory.  One pipeline
// step is one 128-K scale group:
//   warp 0       TMA producer: the 128-token x 128-K activation tile (two 128-byte-swizzled boxes) into a ring in
//                shared memory
//   warps 10..   converters, one thread per weight row and TMEM lane: the row's 64 packed bytes of the group straight
//                from global memory (requested one group ahead), nibble pairs -> bf16 integers by one
//                logic operation and one exact subtraction per pair, re-paired by byte permutes, two tcgen05.st of 32
//                columns into a ring of four A slots.  Two teams of four warps take alternate groups; each keeps
//                two register sets for the packed bytes and alternates between them.
//   warp 1       MMA issuer: 8 x tcgen05.mma kind::f16 (A from tensor memory, 128 x 128 x 16) into one of two
//                accumulators, then ONE commit that tells the converters (A slot free) and the fold warps
//                (accumulator complete), and one for the producer.
// What sets the pace (timestamps written from inside the kernel, and the probe bench/tcgen05_mma_rate.cu): a
// 128 x 128 x 16 MMA with A in tensor memory retires every 93 clocks whatever accumulator it adds to (69 % of the
// dense rate; 128 x 256 x 16: 139 clocks, 92 %), and inside this kernel, beside the converters' tcgen05.st and the
// fold's tcgen05.ld, a group's eight take about twice that.  Wider MMAs are out of reach: two 256-column accumulators
// and the weights do not fit the 512 columns of tensor memory, and every group's accumulator has to be read out for
// its scale.  Measured along the way: 64-K steps were 25 % slower (the issuing thread's chain of waits and commits per
// step); copying the prefetched bytes into a "current" register set cost 0.3 us per group (the copy waits for the
// loads): two sets used alternately, +17 %; a second converter team on top, +15 %; a second issuing thread, a deeper
// activation ring, another tile order and an epilogue staged through shared memory changed nothing.
//   warps 2-9    fold: tcgen05.ld the group's accumulator and add s[n, g] * acc into fp32 registers -- the scale is
//                one scalar per thread and group (lane = weight row); after the last group: bf16, stored transposed.
// Against the form that converts through shared memory (gemm_w4a16_prefill.cu) a group moves 80 KB less through
// shared memory (no converted tile written and read back, no packed tile at all).
// fp32 accumulation inside a group (tensor core) and across groups (registers); one rounding at the end; no product
// q * s is ever rounded ("group-wise partial-sum scaling").
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace w4ts {

constexpr int kRows = 128;           // weight rows per tile (UMMA M, TMEM lanes)
constexpr int kTok = 128;            // tokens per tile (UMMA N)
constexpr int kGroup = 128;          // K per scale group = K per pipeline step
constexpr int kBoxBytes = kTok * 128;        // one 64-K box of activations, 16 KiB
constexpr int kXBytes = 2 * kBoxBytes;       // 32 KiB per step
constexpr int kMaxLoadStages = 6;
constexpr int kASlots = 4;           // ring of converted weight tiles in tensor memory, 64 columns each
constexpr int kFoldWarps = 8, kTeamWarps = 4;
constexpr uint32_t kTmemCols = 512;  // two accumulators of 128 columns + 4 x 64 columns of weights
constexpr int kBarBytes = 256;

struct Params {
    const __nv_bfloat16* X;
    const uint8_t* Wq;
    const __half* S;
    __nv_bfloat16* Y;
    int M, N, K;
    int tiles_m, tiles_n;
    int load_stages;
    uint32_t* status;
};

// (136 + q, 136 + q') as bf16x2 -> (q, q'): exact, both sides are integers below 256
__device__ __forceinline__ uint32_t sub136(uint32_t v)
{
    const uint32_t k = 0x43084308u;
    const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v), *reinterpret_cast<const __nv_bfloat162*>(&k));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// Eight packed words (64 weights of one row) -> 32 words of bf16 pairs in ascending K.
__device__ __forceinline__ void convert64(const uint4& lo, const uint4& hi, uint32_t (&r)[32])
{
    const uint32_t ww[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {                      // word j: K offsets 8 j .. 8 j + 7
        // nibble pairs (i, i + 4) as bf16 integers 136 + q by one logic operation ((w & mask) ^ const flips the sign
        // bit of the nibble and sets the exponent), minus 136 exactly, then pairs of ascending K by byte permutes
        const uint32_t a0 = sub136((ww[j] & 0x000F000Fu) ^ 0x43084308u);
        const uint32_t a1 = sub136(((ww[j] >> 4) & 0x000F000Fu) ^ 0x43084308u);
        const uint32_t a2 = sub136(((ww[j] >> 8) & 0x000F000Fu) ^ 0x43084308u);
        const uint32_t a3 = sub136(((ww[j] >> 12) & 0x000F000Fu) ^ 0x43084308u);
        r[4 * j + 0] = __byte_perm(a0, a1, 0x5410);
        r[4 * j + 1] = __byte_perm(a2, a3, 0x5410);
        r[4 * j + 2] = __byte_perm(a0, a1, 0x7632);
        r[4 * j + 3] = __byte_perm(a2, a3, 0x7632);
    }
}

constexpr int kTeams = 2;          // converter teams: measured 15-20 % over one
__global__ void __launch_bounds__(32 * (2 + kFoldWarps + kTeamWarps * kTeams), 1)
w4a16_prefill_ts_kernel(const __grid_constant__ CUtensorMap tmX, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const int LS = p.load_stages;
    auto x_tile = [&](int s) { return smem_base + s * kXBytes; };
    const uint32_t bar_base = smem_base + LS * kXBytes;
    auto xfull_bar = [&](int s) { return bar_base + 8u * s; };                          // the activation tile has landed
    auto xempty_bar = [&](int s) { return bar_base + 8u * (kMaxLoadStages + s); };      // ... and the MMAs that read it retired
    auto aready_bar = [&](int a) { return bar_base + 8u * (2 * kMaxLoadStages + a); };  // the A slot holds converted weights
    auto done_bar = [&](int a) { return bar_base + 8u * (2 * kMaxLoadStages + kASlots + a); };   // the group's MMAs retired
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kMaxLoadStages + 2 * kASlots + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * kMaxLoadStages + 2 * kASlots + 2);
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.K / kGroup;                              // pipeline steps per tile
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < LS; ++s) { ptx::mbar_init(xfull_bar(s), 1); ptx::mbar_init(xempty_bar(s), 1); }
        for (int a = 0; a < kASlots; ++a) { ptx::mbar_init(aready_bar(a), kTeamWarps); ptx::mbar_init(done_bar(a), 1); }
        for (int b = 0; b < 2; ++b) ptx::mbar_init(tempty_bar(b), kFoldWarps);
        ptx::fence_mbar_init();
    }
    if (warp == 1) { ptx::tmem_alloc(tmem_slot, kTmemCols); ptx::tmem_relinquish(); }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const uint32_t a_tmem0 = tmem_base + 2 * kTok;           // behind the two accumulators

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer: activations
        if (ptx::elect_one()) {
            ptx::tma_prefetch_desc(&tmX);
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / p.tiles_n) * kTok;
                for (int g = 0; g < G; ++g) {
                    if (!ptx::mbar_wait(xempty_bar(stage), phase ^ 1u, p.status, 41)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(xfull_bar(stage), kXBytes);
                    ptx::tma_load_2d(x_tile(stage), &tmX, xfull_bar(stage), g * kGroup, m0);
                    ptx::tma_load_2d(x_tile(stage) + kBoxBytes, &tmX, xfull_bar(stage), g * kGroup + 64, m0);
                    if (++stage == LS) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (ptx::elect_one()) {
            // bf16 x bf16 -> fp32, both K-major; M = 128 weight rows (A, tensor memory), N = 128 tokens (B, shared memory)
            constexpr uint32_t idesc = ptx::umma_idesc(1, 1, kRows, kTok);
            const int total = ((num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)) * G;
            bool ok = true;
            for (int gi = 0; gi < total && ok; ++gi) {               // running group index over all tiles of this CTA
                const int buf = gi & 1, slot = gi & (kASlots - 1), stage = gi % LS;
                if (!ptx::mbar_wait(tempty_bar(buf), ((gi >> 1) & 1u) ^ 1u, p.status, 42) ||
                    !ptx::mbar_wait(xfull_bar(stage), (gi / LS) & 1u, p.status, 43) ||
                    !ptx::mbar_wait(aready_bar(slot), (gi / kASlots) & 1u, p.status, 44)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * kTok;
                const uint32_t a_tmem = a_tmem0 + slot * 64;
                const uint64_t db0 = ptx::smem_desc_sw128_kmajor(x_tile(stage));
                const uint64_t db1 = ptx::smem_desc_sw128_kmajor(x_tile(stage) + kBoxBytes);
#pragma unroll
                for (int k = 0; k < 8; ++k)                         // 16 K: 8 columns of A, 32 bytes of B (+2 in 16-byte units)
                    ptx::umma_f16_ts(d_tmem, a_tmem + 8 * k, (k < 4 ? db0 : db1) + 2u * (k & 3), idesc, k != 0);
                ptx::umma_commit(done_bar(slot));                   // converters: the slot is free; fold: the sum is complete
                ptx::umma_commit(xempty_bar(stage));
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (warp < 2 + kFoldWarps) {
        // ---------------------------------------------------------------- fold: group accumulators -> scaled fp32 sums
        const int q = warp & 3;                                  // TMEM lane quadrant of this warp
        const int half = (warp - 2) >> 2;                        // which 64 of the tile's 128 tokens
        const int row = q * 32 + lane;                           // weight row inside the tile = TMEM lane
        bool ok = true;
        int gi = 0;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile / p.tiles_n) * kTok, n0 = (tile % p.tiles_n) * kRows;
            const int n = n0 + row;
            const __half* srow = p.S + static_cast<size_t>(n < p.N ? n : 0) * G;
            float2 acc[32];                                       // 64 tokens, two per packed fp32 operation
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = make_float2(0.0f, 0.0f);
            float s_next = (n < p.N) ? __half2float(__ldg(srow)) : 0.0f;
            for (int g = 0; g < G && ok; ++g, ++gi) {
                const float s = s_next;
                if (g + 1 < G) s_next = (n < p.N) ? __half2float(__ldg(srow + g + 1)) : 0.0f;
                const int buf = gi & 1, slot = gi & (kASlots - 1);
                if (!ptx::mbar_wait(done_bar(slot), (gi / kASlots) & 1u, p.status, 45)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kTok + 64 * half;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t d[16];
                    ptx::tmem_ld_32x32b_x16(taddr + 16 * c, d);
                    ptx::tmem_ld_wait();
                    if (c == 3) {                                 // all of it is in registers: hand the accumulator back before the arithmetic
                        ptx::tcgen05_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(tempty_bar(buf));
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i)                    // fma.rn.f32x2: the same roundings as two scalar FMAs
                        acc[8 * c + i] = __ffma2_rn(make_float2(__uint_as_float(d[2 * i]), __uint_as_float(d[2 * i + 1])),
                                                    make_float2(s, s), acc[8 * c + i]);
                }
            }
            // one rounding to bf16; the tile is transposed: a warp's lanes are 32 consecutive output columns of one token
            if (ok && n < p.N) {
                __nv_bfloat16* dst = p.Y + static_cast<size_t>(m0 + 64 * half) * p.N + n;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (m0 + 64 * half + 2 * j < p.M) dst[static_cast<size_t>(2 * j) * p.N] = __float2bfloat16_rn(acc[j].x);
                    if (m0 + 64 * half + 2 * j + 1 < p.M) dst[static_cast<size_t>(2 * j + 1) * p.N] = __float2bfloat16_rn(acc[j].y);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- converters: packed int4 -> bf16 A tile in TMEM
        const int team = (warp - 2 - kFoldWarps) >> 2;
        const int row = (warp & 3) * 32 + lane;                  // TMEM lane this warp may write = weight row in the tile
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const size_t row_bytes = static_cast<size_t>(p.K) / 2;
        // position of the bytes requested ahead: (tile, group in tile)
        int pf_tile = blockIdx.x, pf_g = team;
        auto pf_load = [&](uint4 (&w)[4]) {
            while (pf_g >= G) { pf_g -= G; pf_tile += gridDim.x; }
            const int n = (pf_tile % p.tiles_n) * kRows + row;
            if (pf_tile < num_tiles && n < p.N) {
                const uint4* src = reinterpret_cast<const uint4*>(p.Wq + static_cast<size_t>(n) * row_bytes + static_cast<size_t>(pf_g) * (kGroup / 2));
#pragma unroll
                for (int i = 0; i < 4; ++i) w[i] = __ldg(src + i);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) w[i] = make_uint4(0, 0, 0, 0);
            }
            pf_g += kTeams;
        };
        // Two register sets used alternately (the loop is unrolled by two): copying "next" into "current" at the
        // end of a step would wait for the loads just issued, 0.3 us measured per group.
        uint4 wa[4], wb[4];
        pf_load(wa);
        const int total = ((num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)) * G;
        auto step = [&](const uint4 (&cur)[4], uint4 (&nxt)[4], int gi) -> bool {
            const int slot = gi & (kASlots - 1);
            pf_load(nxt);
            if (!ptx::mbar_wait(done_bar(slot), ((gi / kASlots) & 1u) ^ 1u, p.status, 46)) return false;
            ptx::tcgen05_fence_after_sync();
            uint32_t r[32];
            convert64(cur[0], cur[1], r);
            ptx::tmem_st_32x32b_x32(a_tmem0 + lane_addr + slot * 64, r);
            convert64(cur[2], cur[3], r);
            ptx::tmem_st_32x32b_x32(a_tmem0 + lane_addr + slot * 64 + 32, r);
            ptx::tmem_st_wait();
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(aready_bar(slot));
            return true;
        };
        for (int gi = team; gi < total; gi += 2 * kTeams) {       // running group index over all tiles of this CTA
            if (!step(wa, wb, gi)) break;
            if (gi + kTeams < total && !step(wb, wa, gi + kTeams)) break;
        }
    }

    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace w4ts
}  // namespace b200q

namespace b200q {

// Called by b200q_gemm_w4a16 for more than 16 tokens (K a multiple of 128).
int gemm_w4a16_prefill_ts(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int group, void* stream)
{
    using namespace w4ts;
    if (X == nullptr || Wq == nullptr || S == nullptr || Y == nullptr) return cudaErrorInvalidValue;
    if (M <= 0 || N <= 0 || K <= 0 || group != kGroup || K % kGroup != 0) return cudaErrorInvalidValue;
    if (!aligned16(X) || !aligned16(Wq)) return cudaErrorInvalidValue;
    Params p{};
    p.X = static_cast<const __nv_bfloat16*>(X); p.Wq = static_cast<const uint8_t*>(Wq);
    p.S = static_cast<const __half*>(S); p.Y = static_cast<__nv_bfloat16*>(Y);
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + kTok - 1) / kTok; p.tiles_n = (N + kRows - 1) / kRows;
    p.load_stages = kMaxLoadStages;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    CUtensorMap tmX;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
        const uint32_t box[2] = {64, kTok};
        if (encode_tiled(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    const int smem_bytes = 1024 + kBarBytes + p.load_stages * kXBytes;
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
        e = cudaFuncSetAttribute(w4a16_prefill_ts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    w4a16_prefill_ts_kernel<<<grid, 32 * (2 + kFoldWarps + kTeamWarps * kTeams), smem_bytes, st>>>(tmX, p);
    return cudaGetLastError();
}

}  // namespace b200q
