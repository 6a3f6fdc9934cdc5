// tcgen05_mma_kat — known-answer tiles for every tensor-core path of the library, one per reference test program:
//   fp8     op/test/arch_primitives/ptx_mma_fp8.cu:48-59       all-ones E4M3, K = 32            -> 32.0
//   mxfp8   op/test/arch_primitives/ptx_mma_fp8.cu:126-178     the same with UE8M0 scales 1.0   -> 32.0
//   fp4     op/test/arch_primitives/ptx_mma_fp4.cu:49-65,311-324  A = +1.5, B = -0.5, block scales
//           {0.5,1,2,4} x {1,2,0.5,4} over K = 64                                               -> -234 (their -233.75 less C = 0.25)
//   sparse  op/test/arch_primitives/ptx_mma_sparse.cu:128-147,163-184  positions {0,1} kept in every group of four,
//           coordinate-dependent values, exact equality with the dense product
//   int8    op/test/arch_primitives/ptx_mma_integer.cu:50-74,387-401   coordinate formulas, D = A*B + C exact
//   int4    op/test/arch_primitives/ptx_mma_integer.cu:61-74,93-108    S4 weights, low nibble first (W4A16 path, scale 1)
// Every check is exact equality: the inputs are chosen so that all products and sums are exact in fp32 / int32 and
// the results are exact in bf16.  Protocol as the reference's programs: [STAGE] lines, [SUCCESS] / [FAILED], exit 0 / 1.
#include "bench_common.h"
using namespace bench;

template <class T> static std::vector<T> from_device(const T* d, size_t n)
{
    std::vector<T> v(n); CK(cudaMemcpy(v.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost)); return v;
}
static bool all_equal(const std::vector<uint16_t>& c, float want)
{
    for (uint16_t v : c) if (bf16_to_f32(v) != want) return false;
    return true;
}
static bool stage(const char* name, bool ok) { std::printf("[STAGE] %-7s %s\n", name, ok ? "exact" : "MISMATCH"); return ok; }

static bool kat_fp8()
{
    const int M = 16, N = 8, K = 32;
    uint8_t *a = to_device(std::vector<uint8_t>((size_t)M * K, 0x38)), *b = to_device(std::vector<uint8_t>((size_t)N * K, 0x38));
    uint16_t* c; CK(cudaMalloc(&c, M * N * 2));
    CKQ(b200q_gemm_fp8(a, b, c, M, N, K, 1.0f, 1.0f, nullptr)); CK(cudaDeviceSynchronize());
    const bool ok = all_equal(from_device(c, (size_t)M * N), 32.0f);
    cudaFree(a); cudaFree(b); cudaFree(c);
    return stage("fp8", ok);
}

static bool kat_mxfp8()
{
    const int M = 16, N = 8, K = 32;
    uint8_t *a = to_device(std::vector<uint8_t>((size_t)M * K, 0x38)), *b = to_device(std::vector<uint8_t>((size_t)N * K, 0x38));
    uint8_t *sa = to_device(std::vector<uint8_t>(M, 127)), *sb = to_device(std::vector<uint8_t>(N, 127)), *ws;
    CK(cudaMalloc(&ws, b200q_gemm_mxfp8_workspace_bytes(M, N, K)));
    uint16_t* c; CK(cudaMalloc(&c, M * N * 2));
    CKQ(b200q_gemm_mxfp8(a, sa, b, sb, c, M, N, K, ws, nullptr)); CK(cudaDeviceSynchronize());
    const bool ok = all_equal(from_device(c, (size_t)M * N), 32.0f);
    cudaFree(a); cudaFree(b); cudaFree(sa); cudaFree(sb); cudaFree(ws); cudaFree(c);
    return stage("mxfp8", ok);
}

static bool kat_fp4()
{
    const int M = 16, N = 8, K = 64;
    std::vector<uint8_t> sa((size_t)M * 4), sb((size_t)N * 4);
    const uint8_t pa[4] = {0x30, 0x38, 0x40, 0x48}, pb[4] = {0x38, 0x40, 0x30, 0x48};      // UE4M3 0.5 1 2 4 / 1 2 0.5 4
    for (size_t i = 0; i < sa.size(); ++i) sa[i] = pa[i % 4];
    for (size_t i = 0; i < sb.size(); ++i) sb[i] = pb[i % 4];
    uint8_t *a = to_device(std::vector<uint8_t>((size_t)M * K / 2, 0x33)), *b = to_device(std::vector<uint8_t>((size_t)N * K / 2, 0x99));
    uint8_t *dsa = to_device(sa), *dsb = to_device(sb), *ws;
    CK(cudaMalloc(&ws, b200q_gemm_nvfp4_workspace_bytes(M, N, K)));
    uint16_t* c; CK(cudaMalloc(&c, M * N * 2));
    CKQ(b200q_gemm_nvfp4(a, dsa, b, dsb, c, M, N, K, 1.0f, 1.0f, ws, nullptr)); CK(cudaDeviceSynchronize());
    const bool ok = all_equal(from_device(c, (size_t)M * N), -234.0f);
    cudaFree(a); cudaFree(b); cudaFree(dsa); cudaFree(dsb); cudaFree(ws); cudaFree(c);
    return stage("fp4", ok);
}

static bool kat_sparse()
{
    const int M = 16, N = 8, K = 128;
    std::vector<float> dense((size_t)M * K, 0.0f), Bt((size_t)N * K);
    std::vector<uint8_t> comp((size_t)M * K / 2), meta((size_t)M * K / 8, 0x44), Bq((size_t)N * K);     // nibble 0x4: positions 0 and 1
    for (int r = 0; r < M; ++r)
        for (int g = 0; g < K / 4; ++g) {
            const float v0 = float((r + g) % 5 + 1), v1 = -float((r * 2 + g) % 5 + 1);
            dense[(size_t)r * K + 4 * g] = v0; dense[(size_t)r * K + 4 * g + 1] = v1;
            comp[(size_t)r * (K / 2) + 2 * g] = encode_e4m3(v0); comp[(size_t)r * (K / 2) + 2 * g + 1] = encode_e4m3(v1);
        }
    for (int c = 0; c < N; ++c)
        for (int k = 0; k < K; ++k) { Bt[(size_t)c * K + k] = float((k * 3 + c * 5 + 1) % 9 - 4); Bq[(size_t)c * K + k] = encode_e4m3(Bt[(size_t)c * K + k]); }
    uint8_t *dc = to_device(comp), *dm = to_device(meta), *db = to_device(Bq);
    uint16_t* c; CK(cudaMalloc(&c, M * N * 2));
    CKQ(b200q_gemm_sp24_fp8(dc, dm, db, c, M, N, K, 1.0f, 1.0f, nullptr)); CK(cudaDeviceSynchronize());
    const std::vector<uint16_t> got = from_device(c, (size_t)M * N);
    bool ok = true;
    for (int r = 0; r < M; ++r)
        for (int n = 0; n < N; ++n) {
            float acc = 0; for (int k = 0; k < K; ++k) acc += dense[(size_t)r * K + k] * Bt[(size_t)n * K + k];
            ok = ok && bf16_to_f32(got[(size_t)r * N + n]) == bf16_to_f32(f32_to_bf16(acc));
        }
    cudaFree(dc); cudaFree(dm); cudaFree(db); cudaFree(c);
    return stage("sparse", ok);
}

static bool kat_int8()
{
    const int M = 16, N = 8, K = 32;
    std::vector<int8_t> A((size_t)M * K), B((size_t)N * K);
    std::vector<int32_t> C((size_t)M * N);
    for (int r = 0; r < M; ++r) for (int k = 0; k < K; ++k) A[(size_t)r * K + k] = (int8_t)(((r * 3 + k * 5 + 1) % 11) - 5);
    for (int n = 0; n < N; ++n) for (int k = 0; k < K; ++k) B[(size_t)n * K + k] = (int8_t)(((k * 7 + n * 2 + 3) % 9) - 4);
    for (int r = 0; r < M; ++r) for (int n = 0; n < N; ++n) C[(size_t)r * N + n] = r * 13 - n * 5 - 37;
    int8_t *a = to_device(A), *b = to_device(B); int32_t *c = to_device(C), *d; CK(cudaMalloc(&d, M * N * 4));
    CKQ(b200q_gemm_i8(a, b, c, d, M, N, K, nullptr)); CK(cudaDeviceSynchronize());
    const std::vector<int32_t> got = from_device(d, (size_t)M * N);
    bool ok = true;
    for (int r = 0; r < M; ++r)
        for (int n = 0; n < N; ++n) {
            long long acc = C[(size_t)r * N + n];
            for (int k = 0; k < K; ++k) acc += (long long)A[(size_t)r * K + k] * B[(size_t)n * K + k];
            ok = ok && got[(size_t)r * N + n] == (int32_t)acc;
        }
    cudaFree(a); cudaFree(b); cudaFree(c); cudaFree(d);
    return stage("int8", ok);
}

static bool kat_int4()
{
    const int M = 16, N = 8, K = 128;
    std::vector<uint8_t> Wq((size_t)N * K / 2, 0);
    std::vector<uint16_t> X((size_t)M * K), S((size_t)N, f32_to_f16(1.0f));
    std::vector<int> W((size_t)N * K);
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) {
            const int w = ((n * 5 + k * 3 + 2) % 15) - 7;                              // matrix_a_s4_value
            W[(size_t)n * K + k] = w;
            Wq[((size_t)n * K + k) / 2] |= (uint8_t)((w & 0xF) << ((k & 1) * 4));      // low nibble = lower K
        }
    for (int m = 0; m < M; ++m) for (int k = 0; k < K; ++k) X[(size_t)m * K + k] = f32_to_bf16(float(((m * 2 + k * 7 + 4) % 15) - 7));
    uint16_t *x = to_device(X), *s = to_device(S), *y; uint8_t* w = to_device(Wq); CK(cudaMalloc(&y, M * N * 2));
    CKQ(b200q_gemm_w4a16(x, w, s, y, M, N, K, 128, nullptr)); CK(cudaDeviceSynchronize());
    const std::vector<uint16_t> got = from_device(y, (size_t)M * N);
    bool ok = true;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            int acc = 0; for (int k = 0; k < K; ++k) acc += W[(size_t)n * K + k] * (((m * 2 + k * 7 + 4) % 15) - 7);
            ok = ok && bf16_to_f32(got[(size_t)m * N + n]) == bf16_to_f32(f32_to_bf16((float)acc));
        }
    cudaFree(x); cudaFree(s); cudaFree(w); cudaFree(y);
    return stage("int4", ok);
}

int main(int argc, char** argv)
{
    Args a = parse(argc, argv);
    std::printf("[CONFIG] tcgen05_mma_kat: one known-answer tile per tensor-core path%s%s\n", a.case_name.empty() ? "" : ", case ", a.case_name.c_str());
    struct { const char* name; bool (*fn)(); } kats[] = {{"fp8", kat_fp8}, {"mxfp8", kat_mxfp8}, {"fp4", kat_fp4}, {"sparse", kat_sparse},
                                                        {"int8", kat_int8}, {"int4", kat_int4}};
    bool ok = true;
    for (auto& k : kats)
        if (a.case_name.empty() || a.case_name == k.name) ok = k.fn() && ok;
    check_status();
    std::printf(ok ? "[SUCCESS]\n" : "[FAILED]\n");
    return ok ? 0 : 1;
}
