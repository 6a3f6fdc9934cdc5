// gemm_w4a16_bf16 — INT4 weight-only GEMM (group-128 fp16 scales, bf16 activations/out):
// full correctness against the host reference, single-call latency, and streaming bandwidth over
// a stack of distinct weight sets larger than L2 (decode shapes) or TFLOP/s (the prefill shape).
#include "bench_common.h"
using namespace bench;

struct Case { const char* name; int M, N, K; };

static bool run_case(const Case& c, const Args& a)
{
    const int M = c.M, N = c.N, K = c.K, G = K / 128;
    std::printf("[CONFIG] gemm_w4a16_bf16 case=%s M=%d N=%d K=%d group=128 seed=%llu  W int4 U[-8,7], S fp16 U(0.005,0.02), X bf16 N(0,1)\n",
                c.name, M, N, K, (unsigned long long)a.seed);
    std::mt19937_64 rng(a.seed);
    std::vector<uint8_t> Wq((size_t)N * K / 2);
    std::vector<float> Wd((size_t)N * K);
    std::vector<uint16_t> S((size_t)N * G), X((size_t)M * K);
    std::uniform_real_distribution<float> us(0.005f, 0.02f);
    for (auto& s : S) s = f32_to_f16(us(rng));
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; k += 2) {
            const int q0 = (int)(rng() % 16) - 8, q1 = (int)(rng() % 16) - 8;
            Wq[((size_t)n * K + k) / 2] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));       // low nibble = lower K
            Wd[(size_t)n * K + k] = q0 * f16_to_f32(S[(size_t)n * G + k / 128]);
            Wd[(size_t)n * K + k + 1] = q1 * f16_to_f32(S[(size_t)n * G + (k + 1) / 128]);
        }
    std::vector<float> Xf = normal((size_t)M * K, a.seed + 7);
    for (size_t i = 0; i < X.size(); ++i) { X[i] = f32_to_bf16(Xf[i]); Xf[i] = bf16_to_f32(X[i]); }
    const int sets = a.profile ? 2 : (M > 16 ? 8 : 72);        // 72 x 8 MiB of weights > L2
    uint8_t* dW; uint16_t* dS; CK(cudaMalloc(&dW, (size_t)sets * Wq.size())); CK(cudaMalloc(&dS, (size_t)sets * S.size() * 2));
    for (int s = 0; s < sets; ++s) {
        CK(cudaMemcpy(dW + (size_t)s * Wq.size(), Wq.data(), Wq.size(), cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dS + (size_t)s * S.size(), S.data(), S.size() * 2, cudaMemcpyHostToDevice));
    }
    uint16_t *dX = to_device(X), *dY; CK(cudaMalloc(&dY, (size_t)M * N * 2));
    cudaStream_t st; CK(cudaStreamCreate(&st));
    auto launch = [&](int i) {
        const int s = i % sets;
        CKQ(b200q_gemm_w4a16(dX, dW + (size_t)s * Wq.size(), dS + (size_t)s * S.size(), dY, M, N, K, 128, st));
    };
    if (a.profile) { launch(0); launch(1); CK(cudaStreamSynchronize(st)); std::printf("[SUCCESS] profile launch done\n"); return true; }
    launch(0); CK(cudaStreamSynchronize(st));
    std::vector<uint16_t> Y((size_t)M * N); CK(cudaMemcpy(Y.data(), dY, Y.size() * 2, cudaMemcpyDeviceToHost));
    std::vector<float> ref((size_t)M * N);
    auto t0 = std::chrono::steady_clock::now();
    host_gemm_ref(Xf.data(), Wd.data(), ref.data(), M, N, K);
    const double cpu_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::printf("[STAGE] reference: full problem on the host, %.3f s, %.2f GFLOP/s (reference CPU loop)\n", cpu_s, 2.0 * M * N * K / cpu_s / 1e9);
    bool ok = report_errors(compare_bf16(Y.data(), ref.data(), ref.size(), K), "gemm_w4a16_bf16", c.name);
    if (ok && !a.correctness_only) {
        Timing t = time_kernel(launch, st);
        const double bytes = (double)N * K / 2 + (double)N * G * 2 + 2.0 * M * K + 2.0 * M * N;
        const double ms = time_back_to_back(launch, st, 20 * sets);
        std::printf("[BENCHMARK] isolated call latency ms: mean %.4f median %.4f min %.4f\n", t.mean_ms, t.median_ms, t.min_ms);
        std::printf("[BENCHMARK] streaming %d weight sets back to back: %.3f us per call, %.1f GB/s = %.1f %% of measured HBM copy (6453) = %.1f %% of nominal (7700)\n",
                    sets, ms * 1e3, bytes / ms / 1e6, 100 * bytes / ms / 1e6 / 6453, 100 * bytes / ms / 1e6 / 7700);
        if (M > 16) std::printf("[BENCHMARK] %.1f TFLOP/s (2 M N K per call)\n", 2.0 * M * N * K / ms / 1e9);
        std::printf("{\"op\":\"gemm_w4a16_bf16\",\"case\":\"%s\",\"M\":%d,\"N\":%d,\"K\":%d,\"us_per_call\":%.4f,\"gbs\":%.1f,\"tflops\":%.2f}\n", c.name, M, N, K, ms * 1e3, bytes / ms / 1e6, 2.0 * M * N * K / ms / 1e9);
    }
    cudaFree(dW); cudaFree(dS); cudaFree(dX); cudaFree(dY); cudaStreamDestroy(st);
    return ok;
}

int main(int argc, char** argv)
{
    Args a = parse(argc, argv);
    std::vector<Case> cases = {{"decode_m1", 1, 4096, 4096}, {"decode_m16", 16, 4096, 4096}, {"prefill_m512", 512, 4096, 4096}};
    if (a.m > 0 && a.n > 0 && a.k > 0) cases = {{"custom", a.m, a.n, a.k}};
    bool ok = true;
    for (const Case& c : cases)
        if (a.case_name.empty() || a.case_name == c.name) ok = run_case(c, a) && ok;
    std::printf(ok ? "[SUCCESS]\n" : "[FAILED]\n");
    return ok ? 0 : 1;
}
