// gemm_sparse_fp8_bf16 — 2:4 structured-sparse FP8 GEMM, bf16 out: the host side compresses A
// (values + 2-bit positions), the check multiplies the expanded dense A, as the reference's sparse
// test does (op/test/arch_primitives/ptx_mma_sparse.cu:416-434).
#include "bench_common.h"
using namespace bench;

struct Case { const char* name; int M, N, K; };

static bool run_case(const Case& c, const Args& a)
{
    const int M = c.M, N = c.N, K = c.K;
    std::printf("[CONFIG] gemm_sparse_fp8_bf16 case=%s M=%d N=%d K=%d seed=%llu  A: 2 of every 4 K kept (uniform positions), N(0,1); B dense N(0,1); per-tensor scales\n",
                c.name, M, N, K, (unsigned long long)a.seed);
    std::vector<float> A = normal((size_t)M * K, a.seed), B = normal((size_t)N * K, a.seed + 1);
    std::mt19937_64 rng(a.seed + 2);
    static const int pairs[6][2] = {{0, 1}, {0, 2}, {1, 2}, {0, 3}, {1, 3}, {2, 3}};
    std::vector<uint8_t> pick((size_t)M * K / 4);
    for (auto& p : pick) p = (uint8_t)(rng() % 6);
    float ma = 0, mb = 0;
    for (size_t g = 0; g < pick.size(); ++g)
        for (int t = 0; t < 4; ++t) {
            if (t != pairs[pick[g]][0] && t != pairs[pick[g]][1]) A[4 * g + t] = 0.0f;
            ma = std::max(ma, std::fabs(A[4 * g + t]));
        }
    for (float v : B) mb = std::max(mb, std::fabs(v));
    const float sa = ma / 448.0f, sb = mb / 448.0f;
    std::vector<uint8_t> comp((size_t)M * K / 2), meta((size_t)M * K / 8, 0), Bq(B.size());
    for (size_t g = 0; g < pick.size(); ++g) {
        const int p0 = pairs[pick[g]][0], p1 = pairs[pick[g]][1];
        comp[2 * g] = encode_e4m3(A[4 * g + p0] / sa); comp[2 * g + 1] = encode_e4m3(A[4 * g + p1] / sa);
        const uint8_t nib = (uint8_t)(p0 | (p1 << 2));          // ascending pair, lower position in bits [1:0]
        meta[g / 2] |= (g & 1) ? (nib << 4) : nib;
    }
    for (size_t i = 0; i < B.size(); ++i) Bq[i] = encode_e4m3(B[i] / sb);
    uint8_t *dA = to_device(comp), *dE = to_device(meta), *dB = to_device(Bq);
    uint16_t* dC; CK(cudaMalloc(&dC, (size_t)M * N * 2));
    cudaStream_t st; CK(cudaStreamCreate(&st));
    auto launch = [&](int) { CKQ(b200q_gemm_sp24_fp8(dA, dE, dB, dC, M, N, K, sa, sb, st)); };
    if (a.profile) { launch(0); launch(0); CK(cudaStreamSynchronize(st)); check_status(); std::printf("[SUCCESS] profile launch done\n"); return true; }
    launch(0); CK(cudaStreamSynchronize(st)); check_status();
    std::vector<uint16_t> C((size_t)M * N); CK(cudaMemcpy(C.data(), dC, C.size() * 2, cudaMemcpyDeviceToHost));
    const std::vector<int> rows = sample_rows(M, (size_t)M * N * K <= (1ull << 31) ? M : 256, a.seed);
    std::vector<float> Ad(rows.size() * (size_t)K, 0.0f), Bd((size_t)N * K), ref(rows.size() * (size_t)N);
    for (size_t r = 0; r < rows.size(); ++r)
        for (int g = 0; g < K / 4; ++g) {
            const size_t gi = (size_t)rows[r] * (K / 4) + g;
            Ad[r * K + 4 * g + pairs[pick[gi]][0]] = decode_e4m3(comp[2 * gi]) * sa;      // expand to dense
            Ad[r * K + 4 * g + pairs[pick[gi]][1]] = decode_e4m3(comp[2 * gi + 1]) * sa;
        }
    for (size_t i = 0; i < Bd.size(); ++i) Bd[i] = decode_e4m3(Bq[i]) * sb;
    auto t0 = std::chrono::steady_clock::now();
    host_gemm_ref(Ad.data(), Bd.data(), ref.data(), (int)rows.size(), N, K);
    const double cpu_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::vector<uint16_t> got(ref.size());
    for (size_t r = 0; r < rows.size(); ++r) std::memcpy(&got[r * N], &C[(size_t)rows[r] * N], (size_t)N * 2);
    std::printf("[STAGE] reference: %zu of %d rows (dense expanded A) on %u host threads, %.2f s, %.2f GFLOP/s\n",
                rows.size(), M, std::thread::hardware_concurrency(), cpu_s, 2.0 * rows.size() * N * K / cpu_s / 1e9);
    bool ok = report_errors(compare_bf16(got.data(), ref.data(), ref.size(), K), "gemm_sparse_fp8_bf16", c.name);
    if (ok && !a.correctness_only) {
        Timing t = time_kernel(launch, st);
        const double tf = 2.0 * M * N * K / (t.median_ms * 1e-3) / 1e12;
        std::printf("[BENCHMARK] latency ms: mean %.4f median %.4f min %.4f max %.4f stddev %.4f\n", t.mean_ms, t.median_ms, t.min_ms, t.max_ms, t.stddev_ms);
        std::printf("[BENCHMARK] %.1f dense-equivalent TFLOPS  = %.1f %% of nominal sparse FP8 (9000)  = %.1f %% of nominal dense FP8 (4500)\n", tf, 100 * tf / 9000, 100 * tf / 4500);
        std::printf("{\"op\":\"gemm_sparse_fp8_bf16\",\"case\":\"%s\",\"M\":%d,\"N\":%d,\"K\":%d,\"median_ms\":%.5f,\"tflops\":%.2f}\n", c.name, M, N, K, t.median_ms, tf);
        check_status();
    }
    cudaFree(dA); cudaFree(dE); cudaFree(dB); cudaFree(dC); cudaStreamDestroy(st);
    return ok;
}

int main(int argc, char** argv)
{
    Args a = parse(argc, argv);
    std::vector<Case> cases = {{"small", 1024, 1024, 1024}, {"ragged", 1000, 1800, 1408}, {"config", 4096, 8192, 8192}};
    if (a.m > 0 && a.n > 0 && a.k > 0) cases = {{"custom", a.m, a.n, a.k}};
    bool ok = true;
    for (const Case& c : cases)
        if (a.case_name.empty() || a.case_name == c.name) ok = run_case(c, a) && ok;
    std::printf(ok ? "[SUCCESS]\n" : "[FAILED]\n");
    return ok ? 0 : 1;
}
