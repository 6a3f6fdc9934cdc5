// Device helpers shared by the stand-alone all-reduce kernel and the GEMM with the all-reduce
// fused in: system-scope flags with bounded waits, NVSwitch multimem loads/stores, and the
// cross-rank sum of eight partial values.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace b200q {
namespace arc {

using ptx::st_release_sys;
using ptx::ld_acquire_sys;
using ptx::multimem_ld_reduce_f32x4;
using ptx::multimem_ld_reduce_bf16x8;
using ptx::multimem_st_bf16x8;

constexpr int kMaxWorld = 16;

// Bounded wait until *flag has reached `epoch` (flags only grow; the signed difference tolerates
// wrap-around).  On a timeout records (site, block) in *status and returns false.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, uint32_t* status, uint32_t site)
{
    unsigned long long t0 = 0, limit = 0;            // the timer is read only every 64 failed polls
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) < 0) {
        if ((++spins & 0x3Fu) == 0) {
            const unsigned long long now = ptx::globaltimer_ns();
            if (t0 == 0) { t0 = now; limit = ptx::peer_wait_limit_ns(status); }
            else if (now - t0 > limit) {
                atomicCAS(status, 0u, ptx::kStatusTimeout | (site << 24) | (blockIdx.x & 0xFFFFFFu));
                return false;
            }
        }
    }
    return true;
}


// Sum over ranks of eight consecutive partial values starting at element e, returned as eight
// bf16 (one round-to-nearest-even of the fp32 sum).  MC: additions in the switch (their order and
// the rounding of the bf16 form are the hardware's); otherwise plain peer loads added in rank order.
template <bool MC, bool PartialBf16>
__device__ __forceinline__ uint4 reduce8(const void* const* partial_ptrs, const void* partial_mc, int world, long long e)
{
    if (PartialBf16) {
        if (MC) return multimem_ld_reduce_bf16x8(static_cast<const __nv_bfloat16*>(partial_mc) + e);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int r = 0; r < world; ++r) {
            const uint4 x = __ldcg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(partial_ptrs[r]) + e));
            const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { acc[2 * i] += __uint_as_float(w[i] << 16); acc[2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u); }
        }
        return make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                          pack_bf16x2(acc[6], acc[7]));
    }
    float4 a, b;
    if (MC) {
        a = multimem_ld_reduce_f32x4(static_cast<const float*>(partial_mc) + e);
        b = multimem_ld_reduce_f32x4(static_cast<const float*>(partial_mc) + e + 4);
    } else {
        a = make_float4(0.f, 0.f, 0.f, 0.f); b = a;
        for (int r = 0; r < world; ++r) {
            const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(partial_ptrs[r]) + e);
            const float4 x = __ldcg(src), y = __ldcg(src + 1);
            a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
            b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
        }
    }
    return make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
}

// The same sum for U independent groups of eight values at once (elements e[0..U)).  All loads of
// one rank are issued before any addition, so U (x2 for fp32) 16-byte requests per rank are in
// flight per thread: throughput over NVLink comes from the number of outstanding loads.
template <bool MC, bool PartialBf16, int U>
__device__ __forceinline__ void reduce8xU(const void* const* partial_ptrs, const void* partial_mc, int world,
                                          const long long (&e)[U], const bool (&valid)[U], uint4 (&out)[U])
{
    if (MC) {
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (valid[u]) out[u] = reduce8<true, PartialBf16>(partial_ptrs, partial_mc, world, e[u]);
        return;
    }
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;
    for (int r = 0; r < world; ++r) {                  // fixed rank order
        if (PartialBf16) {
            const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(partial_ptrs[r]);
            uint4 x[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                x[u] = valid[u] ? __ldcg(reinterpret_cast<const uint4*>(src + e[u])) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t w[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[u][2 * i] += __uint_as_float(w[i] << 16);
                    acc[u][2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
                }
            }
        } else {
            const float* src = static_cast<const float*>(partial_ptrs[r]);
            float4 x[U], y[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                x[u] = valid[u] ? __ldcg(reinterpret_cast<const float4*>(src + e[u])) : make_float4(0, 0, 0, 0);
                y[u] = valid[u] ? __ldcg(reinterpret_cast<const float4*>(src + e[u]) + 1) : make_float4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                acc[u][0] += x[u].x; acc[u][1] += x[u].y; acc[u][2] += x[u].z; acc[u][3] += x[u].w;
                acc[u][4] += y[u].x; acc[u][5] += y[u].y; acc[u][6] += y[u].z; acc[u][7] += y[u].w;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
        out[u] = make_uint4(pack_bf16x2(acc[u][0], acc[u][1]), pack_bf16x2(acc[u][2], acc[u][3]),
                            pack_bf16x2(acc[u][4], acc[u][5]), pack_bf16x2(acc[u][6], acc[u][7]));
}

template <bool MC>
__device__ __forceinline__ void broadcast8(__nv_bfloat16* const* out_ptrs, __nv_bfloat16* out_mc, int world, long long e, uint4 o)
{
    if (MC) multimem_st_bf16x8(out_mc + e, o);
    else for (int r = 0; r < world; ++r) *reinterpret_cast<uint4*>(out_ptrs[r] + e) = o;
}

}  // namespace arc
}  // namespace b200q
