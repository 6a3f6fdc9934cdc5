// nccl_mlp_test — tensor-parallel SwiGLU MLP on FP8 weights over 1/2/4/8 GPUs of one node.
//
// Keeps the shape of the reference's program of the same name (op/nccl/nccl_mlp_test.cu): one
// process, one stream per device, weights sharded as shard_a / shard_b (:321-352), a sum
// all-reduce of the partial outputs, a single-GPU run of the whole MLP as the reference result
// (build_reference, :208-300), max-abs / max-rel comparison (:444-458), bit-exact replica check
// (:646-664), warm-up + timed iterations with the slowest rank's time reported (:483-526).
// Differences asked for by the benchmark configuration: SwiGLU, E4M3 weights with per-channel
// scales, bf16 activations, --gpus {1,2,4,8}, one host thread per device, and --comm (or B200Q_MLP_COMM):
//   fused      the library's down-projection kernel with the all-reduce fused in (peer loads/stores)
//   pipelined  the library's stand-alone all-reduce kernel on a side stream under the NEXT step's GEMMs,
//              partials and outputs double-buffered (the throughput mode bench.py times; peer loads/stores
//              here: the in-switch transport needs a multicast mapping, which only the Python layer sets up)
//   nccl       b200q GEMMs + ncclAllReduce(bf16, sum) as in the reference
#include <nccl.h>

#include <atomic>
#include <functional>

#include "bench_common.h"
using namespace bench;

#define CKN(x)                                                                         \
    do {                                                                               \
        ncclResult_t r_ = (x);                                                         \
        if (r_ != ncclSuccess) { std::printf("[FAILED] %s: %s\n", #x, ncclGetErrorString(r_)); std::exit(1); } \
    } while (0)

struct Rank {
    int dev = 0;
    cudaStream_t st{}, cs{};                   // GEMM stream, all-reduce side stream (pipelined mode)
    uint8_t *wg{}, *wu{}, *wd{}, *xq{}, *hq{};
    float *sg{}, *su{}, *sd{}, *sx{}, *sh{};
    uint16_t *x{}, *h{}, *partial{}, *y{};
    uint16_t *partial2{}, *y2{};               // second buffers of the pipelined mode
    uint32_t *flags{}, *counters{}, *signals{};
    void **partial_tab{}, **out_tab{}, **flag_tab{};
    void **partial_tab2{}, **out_tab2{}, **signal_tab{};
    cudaEvent_t e0{}, e1{}, gemm_done{}, ar_done[2]{};
    bool ar_used[2] = {false, false};
};

static void run_threads(int n, const std::function<void(int)>& fn)
{
    std::vector<std::thread> th;
    for (int r = 0; r < n; ++r) th.emplace_back(fn, r);
    for (auto& t : th) t.join();
}

int main(int argc, char** argv)
{
    Args a = parse(argc, argv);
    int tokens = 4096, hidden = 8192, inter = 28672;
    std::string comm = "fused";
    if (a.case_name == "small") { tokens = 512; hidden = 1024; inter = 2048; }
    if (a.m > 0) tokens = a.m;
    if (a.n > 0) hidden = a.n;
    if (a.k > 0) inter = a.k;
    if (const char* c = std::getenv("B200Q_MLP_COMM")) comm = c;
    if (!a.comm.empty()) comm = a.comm;
    if (comm != "fused" && comm != "pipelined" && comm != "nccl") { std::printf("[FAILED] --comm must be fused, pipelined or nccl\n"); return 1; }
    const int R = a.gpus;
    int ndev = 0; CK(cudaGetDeviceCount(&ndev));
    if (R < 1 || R > ndev || inter % R != 0) { std::printf("[FAILED] need %d GPUs (have %d) and intermediate %% gpus == 0\n", R, ndev); return 1; }
    const int loc = inter / R;
    std::printf("[CONFIG] nccl_mlp_test tokens=%d hidden=%d intermediate=%d gpus=%d comm=%s seed=%llu  E4M3 weights N(0,1), per-channel scales U(0.001,0.01), bf16 X N(0,1)\n",
                tokens, hidden, inter, R, comm.c_str(), (unsigned long long)a.seed);

    // ---- host data (full, then sharded per rank as the reference's shard_a / shard_b do)
    std::mt19937_64 rng(a.seed);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::uniform_real_distribution<float> ud(0.001f, 0.01f);
    auto rand_w = [&](size_t n) { std::vector<uint8_t> v(n); for (auto& b : v) b = encode_e4m3(nd(rng)); return v; };
    auto rand_s = [&](size_t n) { std::vector<float> v(n); for (auto& s : v) s = ud(rng); return v; };
    std::vector<uint8_t> Wg = rand_w((size_t)inter * hidden), Wu = rand_w((size_t)inter * hidden), Wd = rand_w((size_t)hidden * inter);
    std::vector<float> Sg = rand_s(inter), Su = rand_s(inter), Sd = rand_s(hidden);
    std::vector<uint16_t> X((size_t)tokens * hidden);
    for (auto& v : X) v = f32_to_bf16(nd(rng));

    std::vector<Rank> rk(R + 1);           // rk[R] = the single-GPU reference on device 0
    for (int r = 0; r < R; ++r) rk[r].dev = r;
    rk[R].dev = 0;
    if (R > 1)
        for (int i = 0; i < R; ++i) { CK(cudaSetDevice(i)); for (int j = 0; j < R; ++j) if (i != j) { cudaError_t e = cudaDeviceEnablePeerAccess(j, 0); if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) CK(e); cudaGetLastError(); } }

    auto setup = [&](Rank& k, int rank, int world) {
        CK(cudaSetDevice(k.dev));
        CK(cudaStreamCreateWithFlags(&k.st, cudaStreamNonBlocking));
        CK(cudaEventCreate(&k.e0)); CK(cudaEventCreate(&k.e1));
        const int l = inter / world;
        std::vector<uint8_t> wd((size_t)hidden * l);
        for (int n = 0; n < hidden; ++n) std::memcpy(&wd[(size_t)n * l], &Wd[(size_t)n * inter + (size_t)rank * l], l);   // input-feature slab
        std::vector<uint8_t> wg(Wg.begin() + (size_t)rank * l * hidden, Wg.begin() + (size_t)(rank + 1) * l * hidden);       // output-feature rows
        std::vector<uint8_t> wu(Wu.begin() + (size_t)rank * l * hidden, Wu.begin() + (size_t)(rank + 1) * l * hidden);
        k.wg = to_device(wg); k.wu = to_device(wu); k.wd = to_device(wd);
        k.sg = to_device(std::vector<float>(Sg.begin() + (size_t)rank * l, Sg.begin() + (size_t)(rank + 1) * l));
        k.su = to_device(std::vector<float>(Su.begin() + (size_t)rank * l, Su.begin() + (size_t)(rank + 1) * l));
        k.sd = to_device(Sd); k.x = to_device(X);
        CK(cudaMalloc(&k.xq, (size_t)tokens * hidden)); CK(cudaMalloc(&k.sx, tokens * 4)); CK(cudaMalloc(&k.sh, tokens * 4));
        CK(cudaMalloc(&k.h, (size_t)tokens * l * 2)); CK(cudaMalloc(&k.hq, (size_t)tokens * l));
        CK(cudaMalloc(&k.partial, (size_t)tokens * hidden * 2)); CK(cudaMalloc(&k.y, (size_t)tokens * hidden * 2));
        CK(cudaMalloc(&k.flags, b200q_fused_allreduce_flag_bytes())); CK(cudaMemset(k.flags, 0, b200q_fused_allreduce_flag_bytes()));
        CK(cudaMalloc(&k.counters, b200q_fused_allreduce_counter_bytes()));
        CK(cudaStreamCreateWithFlags(&k.cs, cudaStreamNonBlocking));
        CK(cudaEventCreateWithFlags(&k.gemm_done, cudaEventDisableTiming));
        for (auto& e : k.ar_done) CK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        CK(cudaMalloc(&k.partial2, (size_t)tokens * hidden * 2)); CK(cudaMalloc(&k.y2, (size_t)tokens * hidden * 2));
        CK(cudaMalloc(&k.signals, b200q_allreduce_signal_bytes())); CK(cudaMemset(k.signals, 0, b200q_allreduce_signal_bytes()));
    };
    for (int r = 0; r < R; ++r) setup(rk[r], r, R);
    setup(rk[R], 0, 1);
    // pointer tables: in one process a peer's device pointer is usable directly once peer access is on
    for (int r = 0; r < R; ++r) {
        std::vector<void*> pt(R), ot(R), ft(R);
        for (int j = 0; j < R; ++j) { pt[j] = rk[j].partial; ot[j] = rk[j].y; ft[j] = rk[j].flags; }
        CK(cudaSetDevice(rk[r].dev));
        rk[r].partial_tab = to_device(pt); rk[r].out_tab = to_device(ot); rk[r].flag_tab = to_device(ft);
        for (int j = 0; j < R; ++j) { pt[j] = rk[j].partial2; ot[j] = rk[j].y2; ft[j] = rk[j].signals; }
        rk[r].partial_tab2 = to_device(pt); rk[r].out_tab2 = to_device(ot); rk[r].signal_tab = to_device(ft);
    }
    std::vector<ncclComm_t> comms(R);
    if (comm == "nccl" && R > 1) { std::vector<int> devs(R); for (int i = 0; i < R; ++i) devs[i] = i; CKN(ncclCommInitAll(comms.data(), R, devs.data())); }

    std::atomic<unsigned> epoch{0};
    auto forward = [&](Rank& k, int rank, int world, unsigned ep) {
        const int l = inter / world;
        CKQ(b200q_quant_rows_e4m3(k.x, k.xq, k.sx, tokens, hidden, k.st));
        CKQ(b200q_gemm_fp8_swiglu(k.xq, k.wg, k.wu, k.h, tokens, l, hidden, k.sx, k.sg, k.su, k.st));
        CKQ(b200q_quant_rows_e4m3(k.h, k.hq, k.sh, tokens, l, k.st));
        if (world == 1) CKQ(b200q_gemm_fp8_rowcol(k.hq, k.wd, k.y, tokens, hidden, l, k.sh, k.sd, 0, k.st));
        else if (comm == "fused")
            CKQ(b200q_gemm_fp8_rowcol_allreduce(k.hq, k.wd, k.partial, tokens, hidden, l, k.sh, k.sd, k.partial_tab, k.out_tab,
                                                k.flag_tab, nullptr, nullptr, 1, k.counters, 0, ep, rank, world, k.st));
        else if (comm == "pipelined") {
            const int b = ep & 1;                                   // buffers alternate; the all-reduce of step i runs under step i + 1
            if (k.ar_used[b]) CK(cudaStreamWaitEvent(k.st, k.ar_done[b], 0));   // the all-reduce that last read partial[b] / wrote y[b]
            CKQ(b200q_gemm_fp8_rowcol(k.hq, k.wd, b ? k.partial2 : k.partial, tokens, hidden, l, k.sh, k.sd, 0, k.st));
            CK(cudaEventRecord(k.gemm_done, k.st));
            CK(cudaStreamWaitEvent(k.cs, k.gemm_done, 0));
            CKQ(b200q_allreduce_to_bf16(b ? k.partial_tab2 : k.partial_tab, b ? k.out_tab2 : k.out_tab, k.signal_tab, nullptr, nullptr, 1,
                                        0, (long long)tokens * hidden, rank, world, ep, 0, 148, k.cs));
            CK(cudaEventRecord(k.ar_done[b], k.cs));
            k.ar_used[b] = true;
        } else {
            CKQ(b200q_gemm_fp8_rowcol(k.hq, k.wd, k.y, tokens, hidden, l, k.sh, k.sd, 0, k.st));
            CKN(ncclAllReduce(k.y, k.y, (size_t)tokens * hidden, ncclBfloat16, ncclSum, comms[rank], k.st));
        }
    };
    auto step_all = [&]() {
        const unsigned ep = ++epoch;
        if (comm == "nccl" && R > 1) {                       // one thread drives all ranks, grouped, as the reference does
            CKN(ncclGroupStart());
            for (int r = 0; r < R; ++r) { CK(cudaSetDevice(rk[r].dev)); forward(rk[r], r, R, ep); }
            CKN(ncclGroupEnd());
        } else {
            run_threads(R, [&](int r) { CK(cudaSetDevice(rk[r].dev)); forward(rk[r], r, R, ep); });
        }
    };
    auto sync_all = [&]() { for (int r = 0; r < R; ++r) { CK(cudaSetDevice(rk[r].dev)); CK(cudaStreamSynchronize(rk[r].st)); CK(cudaStreamSynchronize(rk[r].cs)); } };
    // where the result of the step with epoch `ep` lies on a rank
    auto result_of = [&](Rank& k, unsigned ep) { return (comm == "pipelined" && R > 1 && (ep & 1)) ? k.y2 : k.y; };

    if (a.profile) { step_all(); step_all(); sync_all(); std::printf("[SUCCESS] profile launch done\n"); return 0; }

    // ---- correctness: distributed result vs the un-sharded MLP on one GPU, and replica equality
    step_all(); sync_all();
    CK(cudaSetDevice(0)); forward(rk[R], 0, 1, 0); CK(cudaStreamSynchronize(rk[R].st));
    check_status();
    std::vector<uint16_t> ref((size_t)tokens * hidden), y0(ref.size()), yr(ref.size());
    CK(cudaMemcpy(ref.data(), rk[R].y, ref.size() * 2, cudaMemcpyDeviceToHost));
    const unsigned ep_checked = epoch.load();
    CK(cudaSetDevice(rk[0].dev)); CK(cudaMemcpy(y0.data(), result_of(rk[0], ep_checked), y0.size() * 2, cudaMemcpyDeviceToHost));
    bool replicas_equal = true;
    for (int r = 1; r < R; ++r) {
        CK(cudaSetDevice(rk[r].dev)); CK(cudaMemcpy(yr.data(), result_of(rk[r], ep_checked), yr.size() * 2, cudaMemcpyDeviceToHost));
        replicas_equal = replicas_equal && std::memcmp(yr.data(), y0.data(), y0.size() * 2) == 0;
    }
    double num = 0, den = 0; float max_abs = 0, max_rel = 0;
    for (size_t i = 0; i < ref.size(); ++i) {
        const float o = bf16_to_f32(y0[i]), e = bf16_to_f32(ref[i]);
        num += (double)(o - e) * (o - e); den += (double)e * e;
        max_abs = std::max(max_abs, std::fabs(o - e)); max_rel = std::max(max_rel, std::fabs(o - e) / std::max(std::fabs(e), 1e-6f));
    }
    const double fro = std::sqrt(num / std::max(den, 1e-300));
    // With R > 1 each rank quantises its own slice of H on its own per-token grid (E4M3, 3 mantissa
    // bits), so sharded and un-sharded results agree to that quantisation, not bit for bit.
    const bool ok = replicas_equal && (R == 1 ? fro == 0.0 : fro < 5e-2);
    std::printf("[STAGE] correctness vs single-GPU run: rel_frobenius=%.3e max_abs=%.4g max_rel=%.4g  replicas bit-identical: %s\n",
                fro, max_abs, max_rel, replicas_equal ? "yes" : "NO");
    if (!ok) { std::printf("[FAILED]\n"); return 1; }
    if (a.correctness_only) { std::printf("[SUCCESS]\n"); return 0; }

    // ---- benchmark: warm-up, then timed iterations; the slowest rank counts
    const int warmup = 10, iters = 50;
    for (int i = 0; i < warmup; ++i) step_all();
    sync_all();
    for (int r = 0; r < R; ++r) { CK(cudaSetDevice(rk[r].dev)); CK(cudaEventRecord(rk[r].e0, rk[r].st)); }
    for (int i = 0; i < iters; ++i) step_all();
    float worst = 0;
    for (int r = 0; r < R; ++r) {
        CK(cudaSetDevice(rk[r].dev));
        if (comm == "pipelined" && R > 1) { CK(cudaEventRecord(rk[r].gemm_done, rk[r].cs)); CK(cudaStreamWaitEvent(rk[r].st, rk[r].gemm_done, 0)); }   // the last all-reduce counts
        CK(cudaEventRecord(rk[r].e1, rk[r].st)); CK(cudaEventSynchronize(rk[r].e1));
        float ms; CK(cudaEventElapsedTime(&ms, rk[r].e0, rk[r].e1)); worst = std::max(worst, ms);
    }
    check_status();
    const double ms = worst / iters;
    const double flops = 2.0 * tokens * hidden * 2.0 * inter + 2.0 * tokens * (double)inter * hidden;
    std::printf("[BENCHMARK] %.4f ms per forward  %.0f tokens/s  %.1f TFLOPS aggregate over %d GPU(s)\n", ms, tokens / (ms * 1e-3), flops / (ms * 1e-3) / 1e12, R);
    std::printf("{\"op\":\"nccl_mlp_test\",\"gpus\":%d,\"comm\":\"%s\",\"ms\":%.5f,\"tokens_per_s\":%.1f}\n", R, comm.c_str(), ms, tokens / (ms * 1e-3));
    std::printf("[SUCCESS]\n");
    return 0;
}
