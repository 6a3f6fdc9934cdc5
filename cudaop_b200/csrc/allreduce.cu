// Sum all-reduce of the tensor-parallel MLP's partial outputs, written for NVSwitch:
//   Y (bf16, replicated on every rank) = sum over ranks of P_r (fp32 partial of the down projection)
// It takes the place of the in-place ncclAllReduce(ncclFloat, ncclSum) of the reference's
// nccl_mlp_test (op/nccl/nccl_mlp_test.cu:181-195) and keeps its contract: fp32 accumulation and
// bit-identical replicas (each output element is reduced by exactly one rank and then broadcast;
// the reference asserts rank0 == rank1, :646-664).
//
// One kernel per rank, all ranks running it at the same time on their own GPUs:
//   1. start barrier over flags in every rank's signal pad (st.release.sys / ld.acquire.sys);
//   2. rank r reduces elements [r*n/R, (r+1)*n/R): with a multicast mapping one
//      multimem.ld_reduce.add.v4.f32 per 16 bytes lets the switch add the R partials in flight,
//      otherwise R plain peer loads are added in rank order; the fp32 sum is rounded once to bf16
//      and stored to every rank's output (multimem.st, or R peer stores);
//   3. end barrier, so a rank's Y is complete when its kernel ends.
// Plain loads/stores and multimem only: no TMA touches peer memory.  Every flag wait is bounded;
// on a timeout the kernel records it in the status word and returns.
#include "common.cuh"
#include "ptx.cuh"
#include "ar_common.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace ar {

constexpr int kThreads = 512;
constexpr int kMaxWorld = arc::kMaxWorld;
constexpr int kMaxCtas = 256;

struct Params {
    const float* const* partial_ptrs;     // device array [world]: every rank's partial buffer
    __nv_bfloat16* const* out_ptrs;       // device array [world]: every rank's output buffer
    uint32_t* const* signal_ptrs;         // device array [world]: every rank's signal pad
    const float* partial_mc;              // multicast address of the partial buffers, or nullptr
    __nv_bfloat16* out_mc;                // multicast address of the output buffers, or nullptr
    long long offset, elems;              // element range of this call (same on every rank)
    uint32_t epoch;                       // strictly increasing per call, same on every rank
    uint32_t pad_offset_words;            // where this library's flags start inside the signal pad
    int rank, world;
    uint32_t* status;
};

using arc::st_release_sys;
using arc::ld_acquire_sys;

// Barrier between the CTAs with the same index on every rank.  Flags: pad[phase][cta][src_rank].
// Returns false (for the whole CTA) if a peer did not arrive within the cross-rank wait limit.
__device__ __forceinline__ bool rank_barrier(const Params& p, int phase, int cta)
{
    __syncthreads();
    bool ok = true;
    if (threadIdx.x < p.world) {
        const int peer = threadIdx.x;
        const size_t slot = p.pad_offset_words + (static_cast<size_t>(phase) * kMaxCtas + cta) * kMaxWorld;
        __threadfence_system();
        st_release_sys(p.signal_ptrs[peer] + slot + p.rank, p.epoch);
        ok = arc::wait_flag(p.signal_ptrs[p.rank] + slot + peer, p.epoch, p.status, 16u + phase);
    }
    return __syncthreads_and(ok);
}

// The work of CTA `cta` of `nctas` on rank p.rank.  SCATTER: the reduce-scatter half alone — the rank's slice of
// the sum goes to its OWN output buffer only and there is no end barrier; the ranks then complete each other's
// outputs with copy-engine copies ordered behind a b200q_rank_barrier, which take no SM time from a GEMM running
// beside them.
template <bool MC, bool PartialBf16, int UNROLL, bool SCATTER = false>
__device__ __forceinline__ void allreduce_body(const Params& p, int cta, int nctas)
{
    const int nthreads = blockDim.x;          // 128..512: small blocks on every SM disturb a co-running GEMM evenly
    if (!rank_barrier(p, 0, cta)) return;

    const long long per = p.elems / p.world;                 // elements this rank reduces
    const long long base = p.offset + per * p.rank;
    const long long vecs = per / 8;                           // 8 values in -> 8 bf16 (16 bytes) out
    const long long stride = static_cast<long long>(nctas) * nthreads;
    for (long long vb = cta * static_cast<long long>(nthreads) + threadIdx.x; vb < vecs; vb += stride * UNROLL) {
        uint4 o[UNROLL];
        long long e[UNROLL];
        bool valid[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) { valid[u] = vb + u * stride < vecs; e[u] = base + (vb + u * stride) * 8; }
        arc::reduce8xU<MC, PartialBf16, UNROLL>(reinterpret_cast<const void* const*>(p.partial_ptrs), p.partial_mc, p.world,
                                                e, valid, o);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (!valid[u]) continue;
            if (SCATTER) *reinterpret_cast<uint4*>(p.out_ptrs[p.rank] + e[u]) = o[u];
            else arc::broadcast8<MC>(p.out_ptrs, p.out_mc, p.world, e[u], o[u]);
        }
    }
    if (!SCATTER) rank_barrier(p, 1, cta);
}

template <bool MC, bool PartialBf16, int UNROLL>
__global__ void __launch_bounds__(kThreads)
allreduce_to_bf16_kernel(const Params p)
{
    allreduce_body<MC, PartialBf16, UNROLL>(p, blockIdx.x, gridDim.x);
}

template <bool MC, bool PartialBf16>
__global__ void __launch_bounds__(kThreads)
reduce_scatter_to_bf16_kernel(const Params p)
{
    allreduce_body<MC, PartialBf16, 4, true>(p, blockIdx.x, gridDim.x);
}

// Every rank of a small world inside ONE launch on ONE device: CTAs [r * ctas, (r + 1) * ctas) play rank r on
// that rank's buffers (all in this device's memory).  The launch is cooperative, so all CTAs are resident at
// once and the flag protocol between the "ranks" makes progress; separate launches that wait on one another
// on one device would have no such guarantee.  Peer loads/stores only.
template <bool PartialBf16, bool SCATTER>
__global__ void __launch_bounds__(kThreads)
allreduce_one_device_kernel(Params p, int ctas_per_rank)
{
    p.rank = blockIdx.x / ctas_per_rank;
    allreduce_body<false, PartialBf16, 2, SCATTER>(p, blockIdx.x % ctas_per_rank, ctas_per_rank);
}

// out[e] = bf16( sum over i of src_i[e] ), fp32 accumulation in index order, one rounding: the arithmetic of the
// exchange on buffers that all live in this device's memory (the sources were brought here by copy engines).
template <bool PartialBf16>
__global__ void __launch_bounds__(256) sum_to_bf16_kernel(const void* const* srcs, int n, __nv_bfloat16* out, long long elems)
{
    constexpr int U = 4;
    const long long vecs = elems / 8;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long vb = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; vb < vecs; vb += stride * U) {
        uint4 o[U];
        long long e[U];
        bool valid[U];
#pragma unroll
        for (int u = 0; u < U; ++u) { valid[u] = vb + u * stride < vecs; e[u] = (vb + u * stride) * 8; }
        arc::reduce8xU<false, PartialBf16, U>(srcs, nullptr, n, e, valid, o);
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (valid[u]) *reinterpret_cast<uint4*>(out + e[u]) = o[u];
    }
}

// One tiny CTA: a barrier over all ranks on the launching streams (bounded like every other wait).
__global__ void __launch_bounds__(32) rank_barrier_kernel(const Params p)
{
    rank_barrier(p, 0, 0);
}

int g_unroll = 4;
int g_threads = 256;
int g_reserved_smem = 0;   // dynamic shared memory requested only to keep the CTAs off SMs that host a GEMM CTA

}  // namespace ar
}  // namespace b200q

extern "C" {

size_t b200q_allreduce_signal_bytes(void)
{
    return static_cast<size_t>(2) * b200q::ar::kMaxCtas * b200q::ar::kMaxWorld * sizeof(uint32_t);
}

int b200q_allreduce_to_bf16(const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                            void* const* signal_ptrs_dev, const void* partial_multicast, void* out_multicast,
                            int partial_is_bf16, long long elem_offset, long long elems, int rank, int world,
                            unsigned int epoch, unsigned int signal_offset_bytes, int ctas, void* stream)
{
    using namespace b200q;
    if (partial_ptrs_dev == nullptr || out_ptrs_dev == nullptr || signal_ptrs_dev == nullptr) return cudaErrorInvalidValue;
    if (world < 1 || world > ar::kMaxWorld || rank < 0 || rank >= world) return cudaErrorInvalidValue;
    if (elems <= 0 || elem_offset < 0 || elems % (8LL * world) != 0 || elem_offset % 8 != 0) return cudaErrorInvalidValue;
    if (ctas < 1 || ctas > ar::kMaxCtas || signal_offset_bytes % 4 != 0) return cudaErrorInvalidValue;
    if ((partial_multicast == nullptr) != (out_multicast == nullptr)) return cudaErrorInvalidValue;
    ar::Params p{};
    p.partial_ptrs = reinterpret_cast<const float* const*>(partial_ptrs_dev);
    p.out_ptrs = reinterpret_cast<__nv_bfloat16* const*>(out_ptrs_dev);
    p.signal_ptrs = reinterpret_cast<uint32_t* const*>(signal_ptrs_dev);
    p.partial_mc = static_cast<const float*>(partial_multicast);
    p.out_mc = static_cast<__nv_bfloat16*>(out_multicast);
    p.offset = elem_offset; p.elems = elems; p.epoch = epoch; p.pad_offset_words = signal_offset_bytes / 4;
    p.rank = rank; p.world = world;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool mc = partial_multicast != nullptr;
#define B200Q_AR(MC_, BF_, U_)                                                                                   \
    do {                                                                                                        \
        if (ar::g_reserved_smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(ar::allreduce_to_bf16_kernel<MC_, BF_, U_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 ar::g_reserved_smem);                                                          \
        ar::allreduce_to_bf16_kernel<MC_, BF_, U_><<<ctas, ar::g_threads, ar::g_reserved_smem, s>>>(p);          \
    } while (0)
#define B200Q_AR_U(MC_, BF_) do { if (ar::g_unroll >= 8) B200Q_AR(MC_, BF_, 8); else if (ar::g_unroll >= 4) B200Q_AR(MC_, BF_, 4); else if (ar::g_unroll >= 2) B200Q_AR(MC_, BF_, 2); else B200Q_AR(MC_, BF_, 1); } while (0)
    if (partial_is_bf16) { if (mc) B200Q_AR_U(true, true); else B200Q_AR_U(false, true); }
    else { if (mc) B200Q_AR_U(true, false); else B200Q_AR_U(false, false); }
#undef B200Q_AR_U
#undef B200Q_AR
    return cudaGetLastError();
}

int b200q_reduce_scatter_to_bf16(const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                 void* const* signal_ptrs_dev, const void* partial_multicast, int partial_is_bf16,
                                 long long elem_offset, long long elems, int rank, int world, unsigned int epoch,
                                 unsigned int signal_offset_bytes, int ctas, void* stream)
{
    using namespace b200q;
    if (partial_ptrs_dev == nullptr || out_ptrs_dev == nullptr || signal_ptrs_dev == nullptr) return cudaErrorInvalidValue;
    if (world < 1 || world > ar::kMaxWorld || rank < 0 || rank >= world) return cudaErrorInvalidValue;
    if (elems <= 0 || elem_offset < 0 || elems % (8LL * world) != 0 || elem_offset % 8 != 0) return cudaErrorInvalidValue;
    if (ctas < 1 || ctas > ar::kMaxCtas || signal_offset_bytes % 4 != 0) return cudaErrorInvalidValue;
    ar::Params p{};
    p.partial_ptrs = reinterpret_cast<const float* const*>(partial_ptrs_dev);
    p.out_ptrs = reinterpret_cast<__nv_bfloat16* const*>(out_ptrs_dev);
    p.signal_ptrs = reinterpret_cast<uint32_t* const*>(signal_ptrs_dev);
    p.partial_mc = static_cast<const float*>(partial_multicast);
    p.offset = elem_offset; p.elems = elems; p.epoch = epoch; p.pad_offset_words = signal_offset_bytes / 4;
    p.rank = rank; p.world = world;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool mc = partial_multicast != nullptr;
    if (partial_is_bf16) {
        if (mc) ar::reduce_scatter_to_bf16_kernel<true, true><<<ctas, ar::g_threads, 0, s>>>(p);
        else ar::reduce_scatter_to_bf16_kernel<false, true><<<ctas, ar::g_threads, 0, s>>>(p);
    } else {
        if (mc) ar::reduce_scatter_to_bf16_kernel<true, false><<<ctas, ar::g_threads, 0, s>>>(p);
        else ar::reduce_scatter_to_bf16_kernel<false, false><<<ctas, ar::g_threads, 0, s>>>(p);
    }
    return cudaGetLastError();
}

namespace {
int one_device(const void* const* partial_ptrs_dev, void* const* out_ptrs_dev, void* const* signal_ptrs_dev,
               int partial_is_bf16, long long elem_offset, long long elems, int world, unsigned int epoch,
               unsigned int signal_offset_bytes, int ctas_per_rank, bool scatter, void* stream)
{
    using namespace b200q;
    if (partial_ptrs_dev == nullptr || out_ptrs_dev == nullptr || signal_ptrs_dev == nullptr) return cudaErrorInvalidValue;
    if (world < 1 || world > ar::kMaxWorld) return cudaErrorInvalidValue;
    if (elems <= 0 || elem_offset < 0 || elems % (8LL * world) != 0 || elem_offset % 8 != 0) return cudaErrorInvalidValue;
    if (ctas_per_rank < 1 || ctas_per_rank > ar::kMaxCtas || signal_offset_bytes % 4 != 0) return cudaErrorInvalidValue;
    ar::Params p{};
    p.partial_ptrs = reinterpret_cast<const float* const*>(partial_ptrs_dev);
    p.out_ptrs = reinterpret_cast<__nv_bfloat16* const*>(out_ptrs_dev);
    p.signal_ptrs = reinterpret_cast<uint32_t* const*>(signal_ptrs_dev);
    p.offset = elem_offset; p.elems = elems; p.epoch = epoch; p.pad_offset_words = signal_offset_bytes / 4;
    p.rank = 0; p.world = world;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    void* args[2] = {&p, &ctas_per_rank};
    const void* fn = scatter
        ? (partial_is_bf16 ? reinterpret_cast<const void*>(ar::allreduce_one_device_kernel<true, true>)
                           : reinterpret_cast<const void*>(ar::allreduce_one_device_kernel<false, true>))
        : (partial_is_bf16 ? reinterpret_cast<const void*>(ar::allreduce_one_device_kernel<true, false>)
                           : reinterpret_cast<const void*>(ar::allreduce_one_device_kernel<false, false>));
    // cooperative: refused with cudaErrorCooperativeLaunchTooLarge when the CTAs cannot all be resident
    return cudaLaunchCooperativeKernel(fn, dim3(world * ctas_per_rank), dim3(128), args, 0, static_cast<cudaStream_t>(stream));
}
}  // namespace

int b200q_allreduce_to_bf16_one_device(const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                       void* const* signal_ptrs_dev, int partial_is_bf16, long long elem_offset,
                                       long long elems, int world, unsigned int epoch, unsigned int signal_offset_bytes,
                                       int ctas_per_rank, void* stream)
{
    return one_device(partial_ptrs_dev, out_ptrs_dev, signal_ptrs_dev, partial_is_bf16, elem_offset, elems, world, epoch,
                      signal_offset_bytes, ctas_per_rank, false, stream);
}

int b200q_reduce_scatter_to_bf16_one_device(const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                            void* const* signal_ptrs_dev, int partial_is_bf16, long long elem_offset,
                                            long long elems, int world, unsigned int epoch,
                                            unsigned int signal_offset_bytes, int ctas_per_rank, void* stream)
{
    return one_device(partial_ptrs_dev, out_ptrs_dev, signal_ptrs_dev, partial_is_bf16, elem_offset, elems, world, epoch,
                      signal_offset_bytes, ctas_per_rank, true, stream);
}

int b200q_sum_to_bf16(const void* const* srcs_dev, int n, int src_is_bf16, void* out, long long elems, int ctas, void* stream)
{
    using namespace b200q;
    if (srcs_dev == nullptr || out == nullptr || n < 1 || n > ar::kMaxWorld || elems <= 0 || elems % 8 != 0 || !aligned16(out))
        return cudaErrorInvalidValue;
    if (ctas < 1 || ctas > 1024) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (src_is_bf16) ar::sum_to_bf16_kernel<true><<<ctas, 256, 0, s>>>(srcs_dev, n, static_cast<__nv_bfloat16*>(out), elems);
    else ar::sum_to_bf16_kernel<false><<<ctas, 256, 0, s>>>(srcs_dev, n, static_cast<__nv_bfloat16*>(out), elems);
    return cudaGetLastError();
}

size_t b200q_rank_barrier_signal_bytes(void) { return static_cast<size_t>(b200q::ar::kMaxWorld) * sizeof(uint32_t); }

int b200q_rank_barrier(void* const* signal_ptrs_dev, int rank, int world, unsigned int epoch,
                       unsigned int signal_offset_bytes, void* stream)
{
    using namespace b200q;
    if (signal_ptrs_dev == nullptr || world < 1 || world > ar::kMaxWorld || rank < 0 || rank >= world ||
        signal_offset_bytes % 4 != 0)
        return cudaErrorInvalidValue;
    ar::Params p{};
    p.signal_ptrs = reinterpret_cast<uint32_t* const*>(signal_ptrs_dev);
    p.epoch = epoch; p.pad_offset_words = signal_offset_bytes / 4; p.rank = rank; p.world = world;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    ar::rank_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return cudaGetLastError();
}

int b200q_allreduce_set_unroll(int unroll)
{
    if (unroll < 1 || unroll > 8) return cudaErrorInvalidValue;
    b200q::ar::g_unroll = unroll;
    return 0;
}

int b200q_allreduce_set_reserved_smem(int bytes)
{
    if (bytes < 0 || bytes > 200 * 1024) return cudaErrorInvalidValue;
    b200q::ar::g_reserved_smem = bytes;
    return 0;
}

int b200q_allreduce_set_threads(int threads)
{
    if (threads != 128 && threads != 256 && threads != 512) return cudaErrorInvalidValue;
    b200q::ar::g_threads = threads;
    return 0;
}

}  // extern "C"
