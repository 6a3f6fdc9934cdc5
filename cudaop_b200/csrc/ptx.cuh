// Inline-PTX wrappers for sm_100a: mbarrier, TMA (non-multicast), tcgen05 (TMEM
// allocation, UMMA issue/commit, TMEM loads) and the bounded-wait helper.
//
// Convention (as in the reference's op/ptx_utils.cuh, AGENTS.md:23-26): all PTX of
// the library lives here, one wrapper per instruction, each stating the instruction
// it emits; the kernels pull the wrappers they use in with using-declarations.  Every wait is bounded: a wait that runs out records where it gave up in
// a status word and returns false; it never traps and never spins forever.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace ptx {

// Status word layout written on a timed-out wait: bit 31 set, bits [30:24] = site
// id, bits [23:0] = block index (saturated).
constexpr uint32_t kStatusTimeout = 0x80000000u;
// The status word is the first of a small per-device block (defined in common.cu):
//   word 0      status
//   words 2-3   limit, in ns, of waits on something inside this GPU (mbarriers)      default 2 s
//   words 4-5   limit, in ns, of waits on a flag that ANOTHER rank raises            default 10 s
// The limits are settable from the host (b200q_set_wait_limit_ms); kernels read them through the
// status pointer they already carry, and only on the slow path of a wait.
constexpr unsigned long long kDefaultLocalWaitNs = 2000000000ull;
constexpr unsigned long long kDefaultPeerWaitNs = 10000000000ull;
constexpr int kStatusBlockWords = 8;
__device__ __forceinline__ unsigned long long local_wait_limit_ns(const uint32_t* status)
{
    return *reinterpret_cast<const volatile unsigned long long*>(status + 2);
}
__device__ __forceinline__ unsigned long long peer_wait_limit_ns(const uint32_t* status)
{
    return *reinterpret_cast<const volatile unsigned long long*>(status + 4);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t lane_id()
{
    uint32_t l;
    asm volatile("mov.u32 %0, %laneid;" : "=r"(l));
    return l;
}

// elect.sync: one lane of the (converged) warp returns true.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- mbarrier

// mbarrier.init.shared::cta.b64
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// fence.mbarrier_init.release.cluster: makes the inits visible to the async proxy / cluster
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// mbarrier.arrive.expect_tx.shared::cta.b64: one arrival + expected transaction bytes
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// mbarrier.arrive.shared::cta.b64
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// mbarrier.arrive.release.cluster.shared::cluster.b64 on a barrier of any CTA in the cluster
// (address produced by mapa).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// mbarrier.try_wait.parity.shared::cta.b64
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait on a phase parity.  Returns false after the local wait limit, having recorded
// (site, block) in *status.  The caller must then leave its loop and fall through to
// the kernel's tear-down.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t* status, uint32_t site)
{
    if (mbar_try_wait(bar, parity)) return true;
    // The clock is read only every 256 failed polls (a poll itself blocks for a while in hardware), so a
    // wait that ends soon never pays for reading the global timer.
    unsigned long long t0 = 0, limit = 0;
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0xFFu) == 0) {
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0) { t0 = now; limit = local_wait_limit_ns(status); }
            else if (now - t0 > limit) {
                uint32_t b = blockIdx.x > 0xFFFFFFu ? 0xFFFFFFu : blockIdx.x;
                atomicCAS(status, 0u, kStatusTimeout | (site << 24) | b);
                return false;
            }
        }
    }
    return true;
}

// ------------------------------------------------------------------- fences

// fence.proxy.async.shared::cta: generic-proxy smem writes -> visible to the async proxy (TMA/UMMA)
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------- TMA

// prefetch.tensormap: pulls the descriptor (a __grid_constant__ kernel parameter) into cache
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes (no multicast)
// x = innermost coordinate; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* tm, uint32_t bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// cp.async.bulk.tensor.2d.global.shared::cta.bulk_group (store; coordinates must be >= 0)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t smem_src, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_src), "r"(x), "r"(y)
        : "memory");
}
// createpolicy: an L2 eviction-priority descriptor for the cache-hinted forms below
__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// TMA store with an L2 cache hint (results that nobody re-reads soon: evict first, so they do not push
// the operands out of L2)
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* tm, uint32_t smem_src, int x, int y, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;"
        ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_src), "r"(x), "r"(y), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// wait until at most N bulk groups still read their shared-memory source
template <int N>
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// -------------------------------------------------------------------- TMEM

// tcgen05.alloc.cta_group::1: whole-warp, writes the TMEM base address to smem
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ------------------------------------------------------------- descriptors

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128
// bytes with the 128-byte swizzle (what a SWIZZLE_128B TMA box of 128 bytes x rows
// writes): 8-row groups are 1024 bytes apart (stride byte offset), the leading byte
// offset is unused for swizzled K-major (encoded 1), descriptor version 1 (sm_100),
// layout type 2 = SWIZZLE_128B.  The tile base must be 1024-byte aligned; advancing
// along K inside the swizzle row adds the byte offset (>>4) to the start field.
__device__ __forceinline__ uint64_t smem_desc_sw128_kmajor(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);   // start address, bits [0,14)
    d |= static_cast<uint64_t>(1) << 16;                        // leading byte offset (16 B units)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset (16 B units)
    d |= static_cast<uint64_t>(1) << 46;                        // descriptor version
    d |= static_cast<uint64_t>(2) << 61;                        // SWIZZLE_128B
    return d;
}

// Same, for an un-swizzled K-major tile made of 8-row x 16-byte core matrices:
// lbo = byte distance between core matrices adjacent in K, sbo = between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc_noswizzle_kmajor(uint32_t smem_addr, uint32_t lbo, uint32_t sbo)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}

// Instruction descriptor, kind::f8f6f4 / kind::f16 (dense): fp32 accumulate, both
// operands K-major.  Formats for f8f6f4: 0 = E4M3, 1 = E5M2, 5 = E2M1.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n,
                                                  bool sparse = false)
{
    return (sparse ? (1u << 2) : 0u) | (1u << 4) /* D = f32 */ | (a_fmt << 7) | (b_fmt << 10) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Instruction descriptor, kind::i8: signed 8-bit operands (format 1; 0 = unsigned), 32-bit integer accumulator
// (D format 2), both operands K-major, no saturation.
__host__ __device__ constexpr uint32_t umma_idesc_i8(uint32_t m, uint32_t n)
{
    return (2u << 4) /* D = s32 */ | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Instruction descriptor for block-scaled kinds (mxf8f6f4 / mxf4nvf4): no D-format
// field (always f32); scale-factor ids select a byte column inside the 32-bit TMEM
// scale column; scale format 0 = UE4M3, 1 = UE8M0.
__host__ __device__ constexpr uint32_t umma_idesc_block_scaled(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n,
                                                               uint32_t a_sf_id, uint32_t b_sf_id, uint32_t sf_fmt)
{
    return (b_sf_id << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (sf_fmt << 23) |
           ((m >> 4) << 24) | (a_sf_id << 29);
}

// -------------------------------------------------------------------- UMMA

// tcgen05.mma.cta_group::1.kind::f8f6f4  D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// tcgen05.mma.cta_group::2.kind::f8f6f4 (issued by the leader CTA of a pair)
__device__ __forceinline__ void umma_f8f6f4_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// tcgen05.mma.cta_group::1.kind::i8: 8-bit integer operands (signedness per operand in idesc), 32-bit integer
// accumulation in TMEM (exact, wrapping)
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// tcgen05.mma.cta_group::2.kind::i8 (issued by the leader CTA of a pair)
__device__ __forceinline__ void umma_i8_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// tcgen05.mma.cta_group::1.kind::f16 (bf16 / fp16 operands)
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X: E2M1 operands with one
// UE4M3 scale per 16 K-elements, scales read from TMEM.
__device__ __forceinline__ void umma_mxf4nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// tcgen05.mma.sp.cta_group::1.kind::f8f6f4: A is 2:4-compressed, metadata read from TMEM.
__device__ __forceinline__ void umma_sp_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t meta_tmem, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.sp.cta_group::1.kind::f8f6f4 [%0], %1, %2, [%5], %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(meta_tmem)
        : "memory");
}

// tcgen05.commit: the mbarrier receives one arrival when every tcgen05 async operation issued
// so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// cta_group::2 form; cta_mask selects which CTAs of the pair get the arrival (signal multicast, not
// a data load).
__device__ __forceinline__ void umma_commit_2cta(uint32_t bar, uint16_t cta_mask)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(cta_mask)
        : "memory");
}

// tcgen05.cp.cta_group::1.32x128b.warpx4: copies 32 rows x 16 bytes from smem (described by a
// no-swizzle descriptor) into 32 TMEM lanes x 4 columns, replicated to all four lane quadrants.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}
// tcgen05.cp.cta_group::1.128x128b: 128 rows x 16 bytes -> 128 lanes x 4 columns
__device__ __forceinline__ void tmem_cp_128x128b(uint32_t taddr, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// tcgen05.ld.sync.aligned.32x32b.x32.b32: each thread of the warp reads 32 consecutive 32-bit
// columns of its own TMEM lane (lane = 32 * (warp_id % 4) + lane_id).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// tcgen05.ld.sync.aligned.32x32b.x16.b32: 16 consecutive columns of the thread's own lane
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
template <int W> __device__ __forceinline__ void tmem_ld_32x32b(uint32_t taddr, uint32_t (&r)[W]);
template <> __device__ __forceinline__ void tmem_ld_32x32b<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld_32x32b_x32(taddr, r); }
template <> __device__ __forceinline__ void tmem_ld_32x32b<16>(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld_32x32b_x16(taddr, r); }
__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- cluster

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %cluster_ctarank;" : "=r"(r));
    return r;
}
// mapa.shared::cluster: address of the same smem offset in another CTA of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t cta_rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
    return r;
}
// st.shared::cluster.u32: a store into the shared memory of any CTA of the cluster (address from mapa)
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v)
{
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait()
{
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ------------------------------------------------------------ global memory

// ld.global.nc.L1::no_allocate.v4: streaming 16-byte read of data used once
__device__ __forceinline__ uint4 ld_stream_v4(const void* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ------------------------------------------------------ instructions used by single kernels

// st.shared.v4.b32: 16 bytes to a shared-memory address given as a 32-bit shared-window offset
__device__ __forceinline__ void st_shared_v4(uint32_t smem_addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(smem_addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// bar.sync on named barrier 1 for `threads` threads (a subset of the CTA's warps)
template <int kThreads>
__device__ __forceinline__ void named_barrier_1()
{
    asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
}

// cp.async.bulk.tensor.2d with .cta_group::2 (no multicast): completion barrier may be the peer's
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* tm, uint32_t cluster_bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t smem_dst, const CUtensorMap* tm, uint32_t cluster_bar, int x, int y, int z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// tcgen05.cp.cta_group::2.32x128b.warpx4: both CTAs of the pair copy 32 rows x 16 bytes from their own
// shared memory into their own tensor memory
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X: 8-bit (or narrower) float operands with one
// UE8M0 scale per 32 K-elements; the byte of the 32-bit TMEM scale column is chosen by the scale-factor ids of idesc
__device__ __forceinline__ void umma_mxf8f6f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
// tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X
__device__ __forceinline__ void umma_mxf4nvf4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// tcgen05.cp.cta_group::2.128x128b: both CTAs copy 128 rows x 16 bytes from their own shared memory into four
// columns of their own tensor memory
__device__ __forceinline__ void tmem_cp_128x128b_pair(uint32_t taddr, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// tcgen05.mma.sp.cta_group::2.kind::f8f6f4
__device__ __forceinline__ void umma_sp_f8f6f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t meta_tmem, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.sp.cta_group::2.kind::f8f6f4 [%0], %1, %2, [%5], %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(meta_tmem)
        : "memory");
}

// cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes: plain (untiled) bulk copy, no multicast;
// both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// max that returns NaN when either input is NaN (so a NaN activation reaches the exponent test below)
__device__ __forceinline__ float max_nan(float a, float b)
{
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}

// dp4a: four byte products added to a 32-bit accumulator; a unsigned bytes, b unsigned / signed bytes
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// tcgen05.st.sync.aligned.32x32b.x16.b32: 16 consecutive 32-bit columns of the thread's own lane
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// tcgen05.st.sync.aligned.32x32b.x32.b32: each thread writes 32 consecutive columns of its own lane
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// tcgen05.ld.sync.aligned.32x32b.x8.b32
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}

// tcgen05.mma.cta_group::1.kind::f16 with the A operand in tensor memory
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// griddepcontrol: programmatic dependent launch.  launch_dependents lets the next kernel of the
// stream start its own prologue and weight fetch; wait blocks until the previous kernel's
// results (this call's activations) are visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float ld_dsmem_f32(uint32_t cluster_addr)
{
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr));
    return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// multimem.ld_reduce.add.v4.f32: the switch adds the same 16 bytes of every rank's buffer
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc)
{
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
    return v;
}

// multimem.ld_reduce.add.acc::f32.v4.bf16x2: eight bf16 per rank added in the switch
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const __nv_bfloat16* mc)
{
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}

// multimem.st.v4.bf16x2: one 16-byte store delivered to every rank's buffer
__device__ __forceinline__ void multimem_st_bf16x8(__nv_bfloat16* mc, uint4 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

}  // namespace ptx
