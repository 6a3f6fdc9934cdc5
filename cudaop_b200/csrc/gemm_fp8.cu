// Host side of the FP8 GEMM entry points: argument checks, tensor maps, launch.
#include "gemm_fp8.cuh"
#include "../../include/b200q.h"

namespace b200q {
namespace fp8 {

namespace {

template <int EPI, typename OutT>
cudaError_t launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmB2, const Params& p,
                   cudaStream_t stream)
{
    auto kernel = gemm_fp8_kernel<EPI, OutT>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int sms = num_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sms ? tiles : sms;
    kernel<<<grid, kThreads, kSmemBytes, stream>>>(tmA, tmB, tmB2, p);
    return cudaGetLastError();
}

// Shared checks: pointers, positive dims, TMA constraints (16-byte aligned bases, row pitch a
// multiple of 16 bytes).
bool bad_operands(const void* A, const void* B, const void* C, int M, int N, int K)
{
    if (A == nullptr || B == nullptr || C == nullptr) return true;
    if (M <= 0 || N <= 0 || K <= 0) return true;
    if (K % 16 != 0) return true;
    if (!aligned16(A) || !aligned16(B)) return true;
    return false;
}

}  // namespace

cudaError_t gemm(const void* A, const void* B, void* C, int M, int N, int K, int epi, int out_f32, float alpha,
                 const float* row_scale, const float* col_scale, const void* B2, const float* col_scale2,
                 long long ldc, cudaStream_t stream)
{
    if (bad_operands(A, B, C, M, N, K)) return cudaErrorInvalidValue;
    if (epi == kEpiRowCol && (row_scale == nullptr || col_scale == nullptr)) return cudaErrorInvalidValue;
    if (epi == kEpiSwiGLU &&
        (row_scale == nullptr || col_scale == nullptr || col_scale2 == nullptr || B2 == nullptr || !aligned16(B2)))
        return cudaErrorInvalidValue;
    if (ldc < N) return cudaErrorInvalidValue;

    Params p{};
    p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.alpha = alpha;
    p.row_scale = row_scale; p.col_scale = col_scale; p.col_scale2 = col_scale2;
    p.tiles_m = (M + kBM - 1) / kBM;
    p.tiles_n = (epi == kEpiSwiGLU) ? (N + 127) / 128 : (N + kBN - 1) / kBN;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;

    CUtensorMap tmA, tmB, tmB2;
    const uint32_t b_rows = (epi == kEpiSwiGLU) ? 128u : static_cast<uint32_t>(kBN);
    if (!make_tmap_2d_u8(&tmA, A, M, K, K, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    if (!make_tmap_2d_u8(&tmB, B, N, K, K, b_rows, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    tmB2 = tmB;
    if (epi == kEpiSwiGLU &&
        !make_tmap_2d_u8(&tmB2, B2, N, K, K, b_rows, kBK, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;

    switch (epi) {
    case kEpiTensor:
        return out_f32 ? launch<kEpiTensor, float>(tmA, tmB, tmB2, p, stream)
                       : launch<kEpiTensor, __nv_bfloat16>(tmA, tmB, tmB2, p, stream);
    case kEpiRowCol:
        return out_f32 ? launch<kEpiRowCol, float>(tmA, tmB, tmB2, p, stream)
                       : launch<kEpiRowCol, __nv_bfloat16>(tmA, tmB, tmB2, p, stream);
    case kEpiSwiGLU:
        if (out_f32) return cudaErrorInvalidValue;
        return launch<kEpiSwiGLU, __nv_bfloat16>(tmA, tmB, tmB2, p, stream);
    default:
        return cudaErrorInvalidValue;
    }
}

}  // namespace fp8
}  // namespace b200q

extern "C" {

int b200q_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, float scale_a, float scale_b,
                   void* stream)
{
    return b200q::fp8::gemm(A, B, C, M, N, K, b200q::fp8::kEpiTensor, 0, scale_a * scale_b, nullptr, nullptr,
                            nullptr, nullptr, N, static_cast<cudaStream_t>(stream));
}

int b200q_gemm_fp8_rowcol(const void* A, const void* B, void* C, int M, int N, int K, const float* row_scale,
                          const float* col_scale, int out_f32, void* stream)
{
    return b200q::fp8::gemm(A, B, C, M, N, K, b200q::fp8::kEpiRowCol, out_f32, 1.0f, row_scale, col_scale, nullptr,
                            nullptr, N, static_cast<cudaStream_t>(stream));
}

int b200q_gemm_fp8_swiglu(const void* X, const void* Wgate, const void* Wup, void* H, int M, int I, int K,
                          const float* row_scale, const float* gate_scale, const float* up_scale, void* stream)
{
    return b200q::fp8::gemm(X, Wgate, H, M, I, K, b200q::fp8::kEpiSwiGLU, 0, 1.0f, row_scale, gate_scale, Wup,
                            up_scale, I, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
