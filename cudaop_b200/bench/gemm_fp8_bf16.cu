// gemm_fp8_bf16 — FP8 E4M3 GEMM with per-tensor scales, bf16 out: correctness against the host
// restatement of the reference's CPU GEMM on sampled rows, then steady-state timing.
// Cases: config (M=N=K=1024, the reference-runnable configuration), peak (8192^3), ragged.
#include "bench_common.h"
using namespace bench;

struct Case { const char* name; int M, N, K; };

static bool run_case(const Case& c, const Args& a)
{
    const int M = c.M, N = c.N, K = c.K;
    std::printf("[CONFIG] gemm_fp8_bf16 case=%s M=%d N=%d K=%d seed=%llu  A,B: N(0,1) scaled to +-448, E4M3, one fp32 scale each; C bf16\n",
                c.name, M, N, K, (unsigned long long)a.seed);
    std::vector<float> A = normal((size_t)M * K, a.seed), B = normal((size_t)N * K, a.seed + 1);
    float ma = 0, mb = 0;
    for (float v : A) ma = std::max(ma, std::fabs(v));
    for (float v : B) mb = std::max(mb, std::fabs(v));
    const float sa = ma / 448.0f, sb = mb / 448.0f;
    std::vector<uint8_t> Aq(A.size()), Bq(B.size());
    for (size_t i = 0; i < A.size(); ++i) Aq[i] = encode_e4m3(A[i] / sa);
    for (size_t i = 0; i < B.size(); ++i) Bq[i] = encode_e4m3(B[i] / sb);
    uint8_t *dA = to_device(Aq), *dB = to_device(Bq);
    uint16_t* dC; CK(cudaMalloc(&dC, (size_t)M * N * 2));
    cudaStream_t st; CK(cudaStreamCreate(&st));
    auto launch = [&](int) { CKQ(b200q_gemm_fp8(dA, dB, dC, M, N, K, sa, sb, st)); };
    if (a.profile) { launch(0); launch(0); CK(cudaStreamSynchronize(st)); check_status(); std::printf("[SUCCESS] profile launch done\n"); return true; }
    launch(0); CK(cudaStreamSynchronize(st)); check_status();
    std::vector<uint16_t> C((size_t)M * N);
    CK(cudaMemcpy(C.data(), dC, C.size() * 2, cudaMemcpyDeviceToHost));
    // sampled rows against the host reference on the dequantised operands
    const std::vector<int> rows = sample_rows(M, (size_t)M * N * K <= (1ull << 31) ? M : 256, a.seed);
    std::vector<float> Ad(rows.size() * (size_t)K), Bd((size_t)N * K), ref(rows.size() * (size_t)N);
    for (size_t r = 0; r < rows.size(); ++r)
        for (int k = 0; k < K; ++k) Ad[r * K + k] = decode_e4m3(Aq[(size_t)rows[r] * K + k]) * sa;
    for (size_t i = 0; i < Bd.size(); ++i) Bd[i] = decode_e4m3(Bq[i]) * sb;
    auto t0 = std::chrono::steady_clock::now();
    host_gemm_ref(Ad.data(), Bd.data(), ref.data(), (int)rows.size(), N, K);
    const double cpu_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::vector<uint16_t> got(ref.size());
    for (size_t r = 0; r < rows.size(); ++r) std::memcpy(&got[r * N], &C[(size_t)rows[r] * N], (size_t)N * 2);
    std::printf("[STAGE] reference: %zu of %d rows on %u host threads, %.2f s, %.2f GFLOP/s (reference CPU loop)\n",
                rows.size(), M, std::thread::hardware_concurrency(), cpu_s, 2.0 * rows.size() * N * K / cpu_s / 1e9);
    bool ok = report_errors(compare_bf16(got.data(), ref.data(), ref.size(), K), "gemm_fp8_bf16", c.name);
    if (ok && !a.correctness_only) {
        Timing t = time_kernel(launch, st);
        const double tf = 2.0 * M * N * K / (t.median_ms * 1e-3) / 1e12;
        std::printf("[BENCHMARK] latency ms: mean %.4f median %.4f min %.4f max %.4f stddev %.4f\n", t.mean_ms, t.median_ms, t.min_ms, t.max_ms, t.stddev_ms);
        std::printf("[BENCHMARK] %.1f TFLOPS  = %.1f %% of nominal dense FP8 (4500)  = %.1f %% of 2 x measured bf16 burst (3386)\n",
                    tf, 100 * tf / 4500, 100 * tf / 3386);
        std::printf("{\"op\":\"gemm_fp8_bf16\",\"case\":\"%s\",\"M\":%d,\"N\":%d,\"K\":%d,\"median_ms\":%.5f,\"tflops\":%.2f}\n", c.name, M, N, K, t.median_ms, tf);
        check_status();
    }
    cudaFree(dA); cudaFree(dB); cudaFree(dC); cudaStreamDestroy(st);
    return ok;
}

int main(int argc, char** argv)
{
    Args a = parse(argc, argv);
    std::vector<Case> cases = {{"config", 1024, 1024, 1024}, {"ragged", 1000, 1800, 1296}, {"peak", 8192, 8192, 8192}};
    if (a.m > 0 && a.n > 0 && a.k > 0) cases = {{"custom", a.m, a.n, a.k}};
    bool ok = true;
    for (const Case& c : cases)
        if (a.case_name.empty() || a.case_name == c.name) ok = run_case(c, a) && ok;
    std::printf(ok ? "[SUCCESS]\n" : "[FAILED]\n");
    return ok ? 0 : 1;
}
