// gemm_nvfp4_bf16 — NVFP4 block-scaled GEMM (E2M1 data, UE4M3 scale per 16 K, fp32 global
// scales, bf16 out): correctness on sampled rows against the host reference on the dequantised
// operands, then timing.
#include "bench_common.h"
using namespace bench;

struct Case { const char* name; int M, N, K; };

static float decode_ue4m3(uint8_t b) { return decode_e4m3(b & 0x7F); }

static void quantise(const std::vector<float>& x, int R, int K, std::vector<uint8_t>& q, std::vector<uint8_t>& sf, float& g,
                     std::vector<float>* deq)
{
    float mx = 0; for (float v : x) mx = std::max(mx, std::fabs(v));
    g = mx / (6.0f * 448.0f);
    q.assign((size_t)R * K / 2, 0); sf.assign((size_t)R * K / 16, 0);
    if (deq) deq->assign((size_t)R * K, 0.0f);
    for (int r = 0; r < R; ++r)
        for (int b = 0; b < K / 16; ++b) {
            const float* xb = &x[(size_t)r * K + 16 * b];
            float m = 0; for (int t = 0; t < 16; ++t) m = std::max(m, std::fabs(xb[t]));
            const uint8_t s8 = encode_e4m3((m / 6.0f) / g) & 0x7F;
            sf[(size_t)r * (K / 16) + b] = s8;
            const float d = decode_ue4m3(s8) * g;
            for (int t = 0; t < 16; ++t) {
                const uint8_t nib = d > 0 ? encode_e2m1(xb[t] / d) : 0;
                const size_t idx = (size_t)r * K + 16 * b + t;
                q[idx / 2] |= (idx & 1) ? (nib << 4) : nib;
                if (deq) (*deq)[idx] = decode_e2m1(nib) * decode_ue4m3(s8) * g;
            }
        }
}

static bool run_case(const Case& c, const Args& a)
{
    const int M = c.M, N = c.N, K = c.K;
    std::printf("[CONFIG] gemm_nvfp4_bf16 case=%s M=%d N=%d K=%d seed=%llu  N(0,1) -> E2M1, UE4M3 scale per 16 K (max/6), fp32 global scale; C bf16\n",
                c.name, M, N, K, (unsigned long long)a.seed);
    std::vector<float> A = normal((size_t)M * K, a.seed), B = normal((size_t)N * K, a.seed + 1), Bd;
    std::vector<uint8_t> Aq, Bq, sfa, sfb; float ga, gb;
    const std::vector<int> rows = sample_rows(M, (size_t)M * N * K <= (1ull << 31) ? M : 256, a.seed);
    std::vector<float> Adq;
    quantise(A, M, K, Aq, sfa, ga, &Adq);
    quantise(B, N, K, Bq, sfb, gb, &Bd);
    uint8_t *dA = to_device(Aq), *dB = to_device(Bq), *dsa = to_device(sfa), *dsb = to_device(sfb);
    uint8_t *ba, *bb; CK(cudaMalloc(&ba, b200q_nvfp4_sf_bytes(M, K))); CK(cudaMalloc(&bb, b200q_nvfp4_sf_bytes(N, K)));
    uint16_t* dC; CK(cudaMalloc(&dC, (size_t)M * N * 2));
    cudaStream_t st; CK(cudaStreamCreate(&st));
    CKQ(b200q_nvfp4_swizzle_sf(dsa, ba, M, K, st)); CKQ(b200q_nvfp4_swizzle_sf(dsb, bb, N, K, st));
    auto launch = [&](int) { CKQ(b200q_gemm_nvfp4_blocked(dA, ba, dB, bb, dC, M, N, K, ga, gb, st)); };
    if (a.profile) { launch(0); launch(0); CK(cudaStreamSynchronize(st)); check_status(); std::printf("[SUCCESS] profile launch done\n"); return true; }
    launch(0); CK(cudaStreamSynchronize(st)); check_status();
    std::vector<uint16_t> C((size_t)M * N); CK(cudaMemcpy(C.data(), dC, C.size() * 2, cudaMemcpyDeviceToHost));
    std::vector<float> Ad(rows.size() * (size_t)K), ref(rows.size() * (size_t)N);
    for (size_t r = 0; r < rows.size(); ++r) std::memcpy(&Ad[r * K], &Adq[(size_t)rows[r] * K], (size_t)K * 4);
    auto t0 = std::chrono::steady_clock::now();
    host_gemm_ref(Ad.data(), Bd.data(), ref.data(), (int)rows.size(), N, K);
    const double cpu_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::vector<uint16_t> got(ref.size());
    for (size_t r = 0; r < rows.size(); ++r) std::memcpy(&got[r * N], &C[(size_t)rows[r] * N], (size_t)N * 2);
    std::printf("[STAGE] reference: %zu of %d rows on %u host threads, %.2f s, %.2f GFLOP/s (reference CPU loop)\n",
                rows.size(), M, std::thread::hardware_concurrency(), cpu_s, 2.0 * rows.size() * N * K / cpu_s / 1e9);
    bool ok = report_errors(compare_bf16(got.data(), ref.data(), ref.size(), K), "gemm_nvfp4_bf16", c.name);
    if (ok && !a.correctness_only) {
        Timing t = time_kernel(launch, st);
        const double tf = 2.0 * M * N * K / (t.median_ms * 1e-3) / 1e12;
        std::printf("[BENCHMARK] latency ms: mean %.4f median %.4f min %.4f max %.4f stddev %.4f\n", t.mean_ms, t.median_ms, t.min_ms, t.max_ms, t.stddev_ms);
        std::printf("[BENCHMARK] %.1f TFLOPS  = %.1f %% of nominal dense FP4 (9000)  = %.1f %% of 4 x measured bf16 burst (6772)\n", tf, 100 * tf / 9000, 100 * tf / 6772);
        std::printf("{\"op\":\"gemm_nvfp4_bf16\",\"case\":\"%s\",\"M\":%d,\"N\":%d,\"K\":%d,\"median_ms\":%.5f,\"tflops\":%.2f}\n", c.name, M, N, K, t.median_ms, tf);
        check_status();
    }
    cudaFree(dA); cudaFree(dB); cudaFree(dsa); cudaFree(dsb); cudaFree(ba); cudaFree(bb); cudaFree(dC); cudaStreamDestroy(st);
    return ok;
}

int main(int argc, char** argv)
{
    Args a = parse(argc, argv);
    std::vector<Case> cases = {{"small", 1024, 1024, 1024}, {"ragged", 1000, 1800, 1344}, {"config", 8192, 8192, 8192}};
    if (a.m > 0 && a.n > 0 && a.k > 0) cases = {{"custom", a.m, a.n, a.k}};
    bool ok = true;
    for (const Case& c : cases)
        if (a.case_name.empty() || a.case_name == c.name) ok = run_case(c, a) && ok;
    std::printf(ok ? "[SUCCESS]\n" : "[FAILED]\n");
    return ok ? 0 : 1;
}
