// MXFP8 block-scaled GEMM for sm_100a: host entry points and the scale re-layout kernel.
//   C[M,N] (bf16) = (A .* 2^(sfa - 127)) * (B .* 2^(sfb - 127))^T
// A[M,K], B[N,K]: E4M3 bytes; SFA[M,K/32], SFB[N,K/32]: one UE8M0 scale (a biased power of two, 2^(b - 127)) per 32
// consecutive K — the reference's mma ... kind::mxf8f6f4.block_scale.scale_vec::1X semantics
// (op/test/arch_primitives/ptx_mma_fp8.cu:126-178; scale decoder op/test/arch_primitives/ptx_mma_fp6.cu:344-351),
// fp32 accumulate, one round-to-nearest-even cast to bf16 at the end.
// The GEMM itself is the CTA-pair block-scaled kernel of gemm_nvfp4_2cta.cu instantiated for this format
// (tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale, 256 x BN x 32 per instruction).
#include "common.cuh"
#include "../../include/b200q.h"

namespace b200q {

// gemm_nvfp4_2cta.cu
int gemm_block_scaled_pair(int fmt, const void* Aq, const void* SFA_blocked, const void* Bq, const void* SFB_blocked,
                           void* C, int M, int N, int K, float alpha, int bn, void* stream);

namespace mxfp8 {

int g_tile_n = 256;

// Row-major scales [rows, K/32] -> blocked layout [ceil(rows/128)][ceil(K/128)][512 bytes], byte
// (r % 32) * 16 + (r / 32 % 4) * 4 + j for the scale of row r and 32-K step j of the 128-K slab.  Rows beyond `rows`
// and steps beyond K get the byte 0 (2^-127; they multiply operand bytes that the loads zero-fill).
// One thread per output 32-bit word.
__global__ void swizzle_sf_kernel(const uint8_t* __restrict__ src, uint32_t* __restrict__ dst, int rows, int k32, int k128)
{
    const size_t total = static_cast<size_t>((rows + 127) / 128) * k128 * 128;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int w = static_cast<int>(i % 128);          // word inside the block: (r % 32) * 4 + (r / 32)
        const size_t blk = i / 128;
        const int kb = static_cast<int>(blk % k128);
        const int rb = static_cast<int>(blk / k128);
        const int r = rb * 128 + (w >> 2) + 32 * (w & 3);
        uint32_t v = 0;
        if (r < rows) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = 4 * kb + j;
                if (c < k32) v |= static_cast<uint32_t>(src[static_cast<size_t>(r) * k32 + c]) << (8 * j);
            }
        }
        dst[i] = v;
    }
}

}  // namespace mxfp8
}  // namespace b200q

extern "C" {

size_t b200q_mxfp8_sf_bytes(int rows, int K)
{
    if (rows <= 0 || K <= 0 || K % 32 != 0) return 0;
    return static_cast<size_t>((rows + 127) / 128) * ((K + 127) / 128) * 512;
}

int b200q_mxfp8_swizzle_sf(const void* sf_rowmajor, void* sf_blocked, int rows, int K, void* stream)
{
    using namespace b200q;
    if (sf_rowmajor == nullptr || sf_blocked == nullptr || rows <= 0 || K <= 0 || K % 32 != 0) return cudaErrorInvalidValue;
    if (!aligned16(sf_blocked)) return cudaErrorInvalidValue;
    const size_t words = b200q_mxfp8_sf_bytes(rows, K) / 4;
    const int grid = static_cast<int>((words + 255) / 256 < 4096 ? (words + 255) / 256 : 4096);
    mxfp8::swizzle_sf_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(sf_rowmajor), static_cast<uint32_t*>(sf_blocked), rows, K / 32, (K + 127) / 128);
    return cudaGetLastError();
}

int b200q_mxfp8_set_tile_n(int bn)
{
    if (bn != 192 && bn != 256) return cudaErrorInvalidValue;
    b200q::mxfp8::g_tile_n = bn;
    return 0;
}

int b200q_gemm_mxfp8_blocked(const void* A, const void* SFA_blocked, const void* B, const void* SFB_blocked, void* C,
                             int M, int N, int K, void* stream)
{
    return b200q::gemm_block_scaled_pair(1, A, SFA_blocked, B, SFB_blocked, C, M, N, K, 1.0f, b200q::mxfp8::g_tile_n, stream);
}

size_t b200q_gemm_mxfp8_workspace_bytes(int M, int N, int K)
{
    const size_t a = b200q_mxfp8_sf_bytes(M, K), b = b200q_mxfp8_sf_bytes(N, K);
    return (a == 0 || b == 0) ? 0 : a + b;
}

int b200q_gemm_mxfp8(const void* A, const void* SFA, const void* B, const void* SFB, void* C, int M, int N, int K,
                     void* workspace, void* stream)
{
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15u)) return cudaErrorInvalidValue;
    const size_t a_bytes = b200q_mxfp8_sf_bytes(M, K);
    if (a_bytes == 0) return cudaErrorInvalidValue;
    uint8_t* wa = static_cast<uint8_t*>(workspace);
    uint8_t* wb = wa + a_bytes;
    int e = b200q_mxfp8_swizzle_sf(SFA, wa, M, K, stream);
    if (e != 0) return e;
    e = b200q_mxfp8_swizzle_sf(SFB, wb, N, K, stream);
    if (e != 0) return e;
    return b200q_gemm_mxfp8_blocked(A, wa, B, wb, C, M, N, K, stream);
}

}  // extern "C"
