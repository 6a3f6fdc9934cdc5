// gemm_mxfp8_bf16 — MXFP8 block-scaled GEMM (E4M3 data, one UE8M0 scale per 32 K, bf16 out): the known answer of
// the reference's one-instruction test (op/test/arch_primitives/ptx_mma_fp8.cu:126-178: all-ones operands with
// scale 1.0 over K = 32 give 32.0), correctness on sampled rows against the host reference on the dequantised
// operands, then timing.
#include "bench_common.h"
using namespace bench;

struct Case { const char* name; int M, N, K; };

// per 32 K: scale 2^(floor(log2 max) - 8), data e4m3_rn(x / scale)
static void quantise(const std::vector<float>& x, int R, int K, std::vector<uint8_t>& q, std::vector<uint8_t>& sf, std::vector<float>* deq)
{
    q.assign((size_t)R * K, 0); sf.assign((size_t)R * K / 32, 127);
    if (deq) deq->assign((size_t)R * K, 0.0f);
    for (int r = 0; r < R; ++r)
        for (int b = 0; b < K / 32; ++b) {
            const float* xb = &x[(size_t)r * K + 32 * b];
            float m = 0; for (int t = 0; t < 32; ++t) m = std::max(m, std::fabs(xb[t]));
            int e = 127;
            if (m > 0) { int ex; std::frexp(m, &ex); e = std::min(254, std::max(0, ex - 1 - 8 + 127)); }
            sf[(size_t)r * (K / 32) + b] = (uint8_t)e;
            const float inv = std::ldexp(1.0f, 127 - e), sc = std::ldexp(1.0f, e - 127);
            for (int t = 0; t < 32; ++t) {
                const size_t idx = (size_t)r * K + 32 * b + t;
                q[idx] = encode_e4m3(xb[t] * inv);
                if (deq) (*deq)[idx] = decode_e4m3(q[idx]) * sc;
            }
        }
}

static bool known_answer()
{
    const int M = 16, N = 8, K = 32;
    std::vector<uint8_t> A((size_t)M * K, 0x38), B((size_t)N * K, 0x38), sa(M, 127), sb(N, 127);
    uint8_t *dA = to_device(A), *dB = to_device(B), *dsa = to_device(sa), *dsb = to_device(sb), *ws;
    CK(cudaMalloc(&ws, b200q_gemm_mxfp8_workspace_bytes(M, N, K)));
    uint16_t* dC; CK(cudaMalloc(&dC, (size_t)M * N * 2));
    CKQ(b200q_gemm_mxfp8(dA, dsa, dB, dsb, dC, M, N, K, ws, nullptr));
    CK(cudaDeviceSynchronize()); check_status();
    std::vector<uint16_t> C((size_t)M * N); CK(cudaMemcpy(C.data(), dC, C.size() * 2, cudaMemcpyDeviceToHost));
    bool ok = true;
    for (uint16_t v : C) ok = ok && bf16_to_f32(v) == 32.0f;
    std::printf("[STAGE] known answer (all-ones E4M3, UE8M0 1.0, K = 32 -> 32.0 in all %d outputs): %s\n", M * N, ok ? "exact" : "MISMATCH");
    cudaFree(dA); cudaFree(dB); cudaFree(dsa); cudaFree(dsb); cudaFree(ws); cudaFree(dC);
    return ok;
}

static bool run_case(const Case& c, const Args& a)
{
    const int M = c.M, N = c.N, K = c.K;
    std::printf("[CONFIG] gemm_mxfp8_bf16 case=%s M=%d N=%d K=%d seed=%llu  N(0,1) -> E4M3 with UE8M0 scale per 32 K; C bf16\n",
                c.name, M, N, K, (unsigned long long)a.seed);
    std::vector<float> A = normal((size_t)M * K, a.seed), B = normal((size_t)N * K, a.seed + 1), Adq, Bd;
    std::vector<uint8_t> Aq, Bq, sfa, sfb;
    const std::vector<int> rows = sample_rows(M, (size_t)M * N * K <= (1ull << 31) ? M : 256, a.seed);
    quantise(A, M, K, Aq, sfa, &Adq);
    quantise(B, N, K, Bq, sfb, &Bd);
    uint8_t *dA = to_device(Aq), *dB = to_device(Bq), *dsa = to_device(sfa), *dsb = to_device(sfb);
    uint8_t *ba, *bb; CK(cudaMalloc(&ba, b200q_mxfp8_sf_bytes(M, K))); CK(cudaMalloc(&bb, b200q_mxfp8_sf_bytes(N, K)));
    uint16_t* dC; CK(cudaMalloc(&dC, (size_t)M * N * 2));
    cudaStream_t st; CK(cudaStreamCreate(&st));
    CKQ(b200q_mxfp8_swizzle_sf(dsa, ba, M, K, st)); CKQ(b200q_mxfp8_swizzle_sf(dsb, bb, N, K, st));
    auto launch = [&](int) { CKQ(b200q_gemm_mxfp8_blocked(dA, ba, dB, bb, dC, M, N, K, st)); };
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
    bool ok = report_errors(compare_bf16(got.data(), ref.data(), ref.size(), K), "gemm_mxfp8_bf16", c.name);
    if (ok && !a.correctness_only) {
        Timing t = time_kernel(launch, st);
        const double tf = 2.0 * M * N * K / (t.median_ms * 1e-3) / 1e12;
        std::printf("[BENCHMARK] latency ms: mean %.4f median %.4f min %.4f max %.4f stddev %.4f\n", t.mean_ms, t.median_ms, t.min_ms, t.max_ms, t.stddev_ms);
        std::printf("[BENCHMARK] %.1f TFLOPS  = %.1f %% of nominal dense FP8 (4500)  = %.1f %% of 2 x measured bf16 burst (3386)\n", tf, 100 * tf / 4500, 100 * tf / 3386);
        std::printf("{\"op\":\"gemm_mxfp8_bf16\",\"case\":\"%s\",\"M\":%d,\"N\":%d,\"K\":%d,\"median_ms\":%.5f,\"tflops\":%.2f}\n", c.name, M, N, K, t.median_ms, tf);
        check_status();
    }
    cudaFree(dA); cudaFree(dB); cudaFree(dsa); cudaFree(dsb); cudaFree(ba); cudaFree(bb); cudaFree(dC); cudaStreamDestroy(st);
    return ok;
}

int main(int argc, char** argv)
{
    Args a = parse(argc, argv);
    std::vector<Case> cases = {{"small", 1024, 1024, 1024}, {"ragged", 1000, 1800, 1312}, {"peak", 8192, 8192, 8192}};
    if (a.m > 0 && a.n > 0 && a.k > 0) cases = {{"custom", a.m, a.n, a.k}};
    bool ok = a.profile ? true : known_answer();
    for (const Case& c : cases)
        if (a.case_name.empty() || a.case_name == c.name) ok = run_case(c, a) && ok;
    std::printf(ok ? "[SUCCESS]\n" : "[FAILED]\n");
    return ok ? 0 : 1;
}
