// Shared scaffolding of the per-operator benchmark executables.
//
// Each executable follows the reference project's protocol for its test+benchmark programs
// (AGENTS.md:42-44; CLI and statistics modelled on op/conv/opt_conv2d_groups_fp32.cu:706-777,
// 1208-1280): stdout lines [CONFIG] / [STAGE] / [BENCHMARK], a final [SUCCESS] or [FAILED], exit
// code 0 / 1; flags --correctness-only, --case NAME, --profile (one steady-state launch for a
// profiler), --m/--n/--k, --seed.  The correctness stage compares the GPU result with a file-local
// host restatement of the reference's CPU GEMM loop (op/cpu/cpu_ops.cpp:95-114) on sampled rows;
// that host code is the executable's checker only.
#pragma once
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "b200q.h"

#define CK(x)                                                                                     \
    do {                                                                                          \
        cudaError_t e_ = (x);                                                                     \
        if (e_ != cudaSuccess) {                                                                  \
            std::printf("[FAILED] %s: %s\n", #x, cudaGetErrorString(e_));                        \
            std::exit(1);                                                                         \
        }                                                                                         \
    } while (0)
#define CKQ(x)                                                                                    \
    do {                                                                                          \
        int e_ = (x);                                                                             \
        if (e_ != 0) {                                                                            \
            std::printf("[FAILED] %s returned cudaError %d\n", #x, e_);                          \
            std::exit(1);                                                                         \
        }                                                                                         \
    } while (0)

namespace bench {

struct Args {
    bool correctness_only = false, profile = false;
    std::string case_name, comm;
    int m = 0, n = 0, k = 0, gpus = 1;
    uint64_t seed = 0;
};

inline Args parse(int argc, char** argv)
{
    Args a;
    for (int i = 1; i < argc; ++i) {
        std::string s = argv[i];
        auto next = [&]() { return (i + 1 < argc) ? std::string(argv[++i]) : std::string(); };
        if (s == "--correctness-only") a.correctness_only = true;
        else if (s == "--profile") a.profile = true;
        else if (s == "--case") a.case_name = next();
        else if (s == "--m") a.m = std::atoi(next().c_str());
        else if (s == "--n") a.n = std::atoi(next().c_str());
        else if (s == "--k") a.k = std::atoi(next().c_str());
        else if (s == "--gpus") a.gpus = std::atoi(next().c_str());
        else if (s == "--comm") a.comm = next();
        else if (s == "--seed") a.seed = std::strtoull(next().c_str(), nullptr, 10);
        else { std::printf("usage: %s [--correctness-only] [--case NAME] [--profile] [--m M --n N --k K] [--seed S] [--gpus G --comm MODE]\n", argv[0]); std::exit(2); }
    }
    return a;
}

// ---------------------------------------------------------------- host codecs (checker side)
inline float decode_e4m3(uint8_t b)
{
    const int e = (b >> 3) & 15, m = b & 7;
    float v = (e == 0) ? std::ldexp(m / 8.0f, -6) : std::ldexp(1.0f + m / 8.0f, e - 7);
    if ((b & 0x7F) == 0x7F) v = NAN;
    return (b & 0x80) ? -v : v;
}
inline uint8_t encode_e4m3(float f)
{
    const uint8_t s = std::signbit(f) ? 0x80 : 0;
    const float a = std::fabs(f);
    if (std::isnan(f)) return 0x7F;
    if (a < std::ldexp(1.0f, -6)) return s | static_cast<uint8_t>(std::nearbyint(std::ldexp(a, 9)));
    if (a > 448.0f) return s | 0x7E;
    int e; const float m = std::frexp(a, &e);
    int q = static_cast<int>(std::nearbyint((m * 2.0f - 1.0f) * 8.0f)); e -= 1;
    if (q == 8) { q = 0; e += 1; }
    if (e > 8 || (e == 8 && q > 6)) return s | 0x7E;
    return s | static_cast<uint8_t>(((e + 7) << 3) | q);
}
inline float decode_e2m1(uint8_t n)
{
    static const float mag[8] = {0, 0.5f, 1, 1.5f, 2, 3, 4, 6};
    return (n & 8) ? -mag[n & 7] : mag[n & 7];
}
inline uint8_t encode_e2m1(float f)
{
    const uint8_t s = std::signbit(f) ? 8 : 0;
    const float a = std::fabs(f);
    uint8_t c;
    if (a <= 0.25f) c = 0; else if (a < 0.75f) c = 1; else if (a <= 1.25f) c = 2; else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4; else if (a < 3.5f) c = 5; else if (a <= 5.0f) c = 6; else c = 7;
    return s | c;
}
inline float bf16_to_f32(uint16_t h) { uint32_t u = static_cast<uint32_t>(h) << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline uint16_t f32_to_bf16(float f)
{
    uint32_t u; std::memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
inline uint16_t f32_to_f16(float f)
{
    const uint16_t s = std::signbit(f) ? 0x8000 : 0;
    const float a = std::fabs(f);
    if (a < std::ldexp(1.0f, -14)) return s | static_cast<uint16_t>(std::nearbyint(std::ldexp(a, 24)));
    int e; const float m = std::frexp(a, &e);
    int q = static_cast<int>(std::nearbyint((m * 2.0f - 1.0f) * 1024.0f)); e -= 1;
    if (q == 1024) { q = 0; e += 1; }
    return s | static_cast<uint16_t>(((e + 15) << 10) | q);
}
inline float f16_to_f32(uint16_t h)
{
    const int e = (h >> 10) & 31, m = h & 1023;
    const float v = (e == 0) ? std::ldexp(static_cast<float>(m), -24) : std::ldexp(1.0f + m / 1024.0f, e - 15);
    return (h & 0x8000) ? -v : v;
}

// C[rows,N] = A[rows,K] * B[N,K]^T with the reference loop (sequential fp32 sum, K innermost),
// spread over host threads by row blocks.
inline void host_gemm_ref(const float* A, const float* B, float* C, int rows, int N, int K)
{
    const int nt = std::max(1u, std::min<unsigned>(std::thread::hardware_concurrency(), rows));
    std::vector<std::thread> th;
    for (int t = 0; t < nt; ++t)
        th.emplace_back([=]() {
            for (int i = t; i < rows; i += nt)
                for (int j = 0; j < N; ++j) {
                    float acc = 0.0f;
                    for (int p = 0; p < K; ++p) acc += A[static_cast<size_t>(i) * K + p] * B[static_cast<size_t>(j) * K + p];
                    C[static_cast<size_t>(i) * N + j] = acc;
                }
        });
    for (auto& t : th) t.join();
}

struct ErrorStats { double rel_fro = 0, rel_fro_raw = 0, max_ulp_floor = 0, max_ulp_strict = 0; long violators = 0; size_t n = 0; };

// The acceptance metrics on a row sample: Frobenius error against the reference given the same
// final bf16 cast, and the bf16-ulp distance to the fp32 reference with the reference's own
// summation-noise floor (4 eps sqrt(K) rms).
inline ErrorStats compare_bf16(const uint16_t* out, const float* ref, size_t n, int K)
{
    double num = 0, num_raw = 0, den = 0, sq = 0;
    for (size_t i = 0; i < n; ++i) sq += static_cast<double>(ref[i]) * ref[i];
    const double rms = std::sqrt(sq / std::max<size_t>(n, 1));
    const double noise = 4.0 * std::ldexp(1.0, -24) * std::sqrt(static_cast<double>(K)) * rms;
    ErrorStats s;
    for (size_t i = 0; i < n; ++i) {
        const double o = bf16_to_f32(out[i]), r = ref[i], rb = bf16_to_f32(f32_to_bf16(ref[i]));
        num += (o - rb) * (o - rb); num_raw += (o - r) * (o - r); den += r * r;
        const double ulp = std::ldexp(1.0, static_cast<int>(std::floor(std::log2(std::max(std::fabs(r), 1e-37)))) - 7);
        const double d = std::fabs(o - r);
        if (d / ulp > 2.0) ++s.violators;
        s.max_ulp_strict = std::max(s.max_ulp_strict, d / ulp);
        s.max_ulp_floor = std::max(s.max_ulp_floor, std::max(d - noise, 0.0) / ulp);
    }
    s.rel_fro = std::sqrt(num / std::max(den, 1e-300));
    s.rel_fro_raw = std::sqrt(num_raw / std::max(den, 1e-300));
    s.n = n;
    return s;
}

// Prints the acceptance metrics and, as one JSON line, the strict figures beside them (the Frobenius error
// against the UNROUNDED fp32 reference, the largest strict ulp distance and the count of elements beyond 2
// ulp without the noise floor), so what the two definitions above set aside stays visible.
inline bool report_errors(const ErrorStats& e, const char* op = "", const char* case_name = "")
{
    std::printf("[STAGE] correctness: rel_frobenius=%.3e (bar 1e-3)  max_bf16_ulp=%.3f (bar 2, noise floor applied)  "
                "strict_2ulp_violators=%ld\n", e.rel_fro, e.max_ulp_floor, e.violators);
    std::printf("{\"op\":\"%s\",\"case\":\"%s\",\"parity\":{\"elements\":%zu,\"rel_fro\":%.4e,\"rel_fro_raw\":%.4e,"
                "\"max_ulp_floor\":%.4f,\"max_ulp_strict\":%.3f,\"violators_2ulp\":%ld}}\n",
                op, case_name, e.n, e.rel_fro, e.rel_fro_raw, e.max_ulp_floor, e.max_ulp_strict, e.violators);
    return e.rel_fro <= 1e-3 && e.max_ulp_floor <= 2.0;
}

struct Timing { double mean_ms, median_ms, min_ms, max_ms, stddev_ms; };

// 3 groups x (warm-up, samples); each sample is one launch between two events on the stream.
template <class F>
Timing time_kernel(F&& launch, cudaStream_t stream, int groups = 3, int warmup = 20, int samples = 100)
{
    std::vector<double> all;
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int g = 0; g < groups; ++g) {
        for (int i = 0; i < warmup; ++i) launch(i);
        CK(cudaStreamSynchronize(stream));
        for (int i = 0; i < samples; ++i) {
            CK(cudaEventRecord(e0, stream)); launch(i); CK(cudaEventRecord(e1, stream));
            CK(cudaEventSynchronize(e1));
            float ms; CK(cudaEventElapsedTime(&ms, e0, e1)); all.push_back(ms);
        }
    }
    std::sort(all.begin(), all.end());
    double sum = 0; for (double v : all) sum += v;
    const double mean = sum / all.size();
    double var = 0; for (double v : all) var += (v - mean) * (v - mean);
    CK(cudaEventDestroy(e0)); CK(cudaEventDestroy(e1));
    return {mean, all[all.size() / 2], all.front(), all.back(), std::sqrt(var / all.size())};
}

// `iters` launches back to back between one pair of events: steady-state time per launch.
template <class F>
double time_back_to_back(F&& launch, cudaStream_t stream, int iters, int warmup = 20)
{
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int i = 0; i < warmup; ++i) launch(i);
    CK(cudaStreamSynchronize(stream));
    CK(cudaEventRecord(e0, stream));
    for (int i = 0; i < iters; ++i) launch(i);
    CK(cudaEventRecord(e1, stream)); CK(cudaEventSynchronize(e1));
    float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
    CK(cudaEventDestroy(e0)); CK(cudaEventDestroy(e1));
    return ms / iters;
}

inline void check_status()
{
    unsigned int st = 0;
    CKQ(b200q_status(&st, 1));
    if (st != 0) { std::printf("[FAILED] a kernel gave up on a bounded wait, status word 0x%08x\n", st); std::exit(1); }
}

template <class T>
T* to_device(const std::vector<T>& v)
{
    T* d = nullptr;
    CK(cudaMalloc(&d, std::max<size_t>(v.size(), 1) * sizeof(T)));
    CK(cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}

inline std::vector<float> normal(size_t n, uint64_t seed)
{
    std::mt19937_64 rng(seed);
    std::normal_distribution<float> d(0.0f, 1.0f);
    std::vector<float> v(n);
    for (auto& x : v) x = d(rng);
    return v;
}

inline std::vector<int> sample_rows(int M, int count, uint64_t seed)
{
    std::mt19937_64 rng(seed ^ 0x9E3779B97F4A7C15ull);
    std::vector<int> r;
    count = std::min(count, M);
    if (count == M) { for (int i = 0; i < M; ++i) r.push_back(i); return r; }
    std::vector<char> used(M, 0);
    while (static_cast<int>(r.size()) < count) {
        int i = static_cast<int>(rng() % M);
        if (!used[i]) { used[i] = 1; r.push_back(i); }
    }
    return r;
}

}  // namespace bench
