// tcgen05_mma_rate — how fast one SM retires back-to-back tcgen05.mma kind::f16 instructions, by shape and by
// whether consecutive instructions add to the same accumulator.  An architecture probe in the manner of the
// reference's op/test/dram_bandwidth.cu (one number per configuration, measured on the device), kept because the
// prefill W4A16 kernels are bounded by exactly this: their scale groups force 128-column accumulators.
//   chain     every MMA accumulates onto the tile the previous one wrote (what a K loop does)
//   alternate consecutive MMAs go to two different accumulators
// Operands are zero-filled shared-memory tiles (128-byte swizzle, K-major) or, for "ts", tensor memory as the A
// operand; 256 instructions are issued by one thread, one commit, the clock is read before the first issue and
// after the commit's barrier has completed.  Output: clocks per instruction and the fraction of the dense bf16
// rate (8192 flop per clock and SM).  [STAGE] lines, [SUCCESS], exit 0; no known answer to compare with.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <cuda_runtime.h>
#include "../csrc/ptx.cuh"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("[FAILED] %s: %s\n", #x, cudaGetErrorString(e_)); std::exit(1); } } while (0)

constexpr int kInstr = 256;

// mode bits: 0 = alternate accumulators, 1 = A operand from tensor memory
template <int N>
__global__ void __launch_bounds__(128, 1) rate_kernel(int mode, long long* clocks, int* gave_up)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - ptx::smem_u32(smem_raw));
    const uint32_t a_tile = base, b_tile = base + 16384;            // 128 x 64 bf16, N x 64 bf16
    const uint32_t bar = b_tile + N * 128, slot = bar + 8;
    for (int i = threadIdx.x; i < (16384 + N * 128) / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(gen)[i] = make_uint4(0, 0, 0, 0);
    ptx::fence_proxy_async_smem();
    if (threadIdx.x == 0) { ptx::mbar_init(bar, 1); ptx::fence_mbar_init(); }
    if (threadIdx.x < 32) { ptx::tmem_alloc(slot, 512); ptx::tmem_relinquish(); }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(gen + (slot - base));
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = ptx::umma_idesc(1, 1, 128, N);
        const uint64_t da = ptx::smem_desc_sw128_kmajor(a_tile), db = ptx::smem_desc_sw128_kmajor(b_tile);
        const bool alt = mode & 1, ts = mode & 2;
        const uint32_t a_tmem = tmem + 480;                         // 32 columns of (uninitialised) bf16 pairs
        const long long t0 = clock64();
        for (int i = 0; i < kInstr; ++i) {
            const uint32_t d = tmem + ((alt && (i & 1)) ? N : 0);
            const int k = i & 3;                                     // the four 16-K slices of the tile, over and over
            if (ts) ptx::umma_f16_ts(d, a_tmem + 8 * k, db + 2u * k, idesc, i >= 2);
            else ptx::umma_f16(d, da + 2u * k, db + 2u * k, idesc, i >= 2);
        }
        ptx::umma_commit(bar);
        int spins = 0;
        while (!ptx::mbar_try_wait(bar, 0) && ++spins < (1 << 22)) {}
        const long long t1 = clock64();
        if (spins >= (1 << 22)) *gave_up = 1;
        clocks[blockIdx.x] = t1 - t0;
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) { ptx::tcgen05_fence_after_sync(); ptx::tmem_dealloc(tmem, 512); }
}

template <int N> static void run(const char* what, int mode, int sms, long long* d_clocks, int* d_flag)
{
    const int smem = 1024 + 16384 + N * 128 + 64;
    CK(cudaFuncSetAttribute(rate_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    for (int rep = 0; rep < 3; ++rep) rate_kernel<N><<<sms, 128, smem>>>(mode, d_clocks, d_flag);
    CK(cudaDeviceSynchronize());
    std::vector<long long> c(sms);
    CK(cudaMemcpy(c.data(), d_clocks, sms * sizeof(long long), cudaMemcpyDeviceToHost));
    std::sort(c.begin(), c.end());
    const double per = double(c[sms / 2]) / kInstr;
    const double ideal = 128.0 * N * 16 * 2 / 8192.0;
    std::printf("[STAGE] 128 x %3d x 16 %-28s %7.1f clocks per instruction (arithmetic alone: %5.1f) -> %5.1f %% of the dense bf16 rate\n",
                N, what, per, ideal, 100.0 * ideal / per);
}

int main()
{
    int dev = 0, sms = 0;
    CK(cudaGetDevice(&dev));
    CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    std::printf("[CONFIG] tcgen05_mma_rate: %d instructions per SM on %d SMs, kind::f16, bf16 operands, fp32 accumulators\n", kInstr, sms);
    long long* d_clocks; int* d_flag;
    CK(cudaMalloc(&d_clocks, sms * sizeof(long long))); CK(cudaMalloc(&d_flag, sizeof(int))); CK(cudaMemset(d_flag, 0, sizeof(int)));
    run<64>("chain", 0, sms, d_clocks, d_flag);
    run<64>("alternate", 1, sms, d_clocks, d_flag);
    run<128>("chain", 0, sms, d_clocks, d_flag);
    run<128>("alternate", 1, sms, d_clocks, d_flag);
    run<128>("chain, A in tensor memory", 2, sms, d_clocks, d_flag);
    run<128>("alternate, A in tensor memory", 3, sms, d_clocks, d_flag);
    run<256>("chain", 0, sms, d_clocks, d_flag);
    run<256>("chain, A in tensor memory", 2, sms, d_clocks, d_flag);
    int flag = 0;
    CK(cudaMemcpy(&flag, d_flag, sizeof(int), cudaMemcpyDeviceToHost));
    cudaFree(d_clocks); cudaFree(d_flag);
    if (flag) { std::printf("[FAILED] a wait ran out\n"); return 1; }
    std::printf("[SUCCESS]\n");
    return 0;
}
