// Host side of the FP8 GEMM entry points: argument checks, tile choice, tensor maps, launch.
#include "gemm_fp8.cuh"
#include "gemm_fp8_2cta.cuh"
#include "../../include/b200q.h"

#include <mutex>

namespace b200q {
namespace fp8 {

namespace {

int g_force_bn = 0;      // 0 = choose per problem; 224 or 256 = forced (b200q_fp8_set_tile_n)
int g_pair_group = 0;    // CTA-pair kernels: tile rows (of 256) that walk the N tiles together; 0 = by L2 footprint (b200q_fp8_set_group)
int g_reducer_stride = 1;
int g_sm_limit = 0;       // 0 = all SMs; otherwise the persistent grids use at most this many (b200q_fp8_set_sm_limit)

int usable_sms()
{
    const int n = num_sms();
    return (g_sm_limit > 0 && g_sm_limit < n) ? g_sm_limit : n;
}
int g_dynamic_tiles = 1;  // CTA-pair kernels take their tiles from a global counter (b200q_fp8_set_dynamic_tiles)
int g_tma_store = 1;     // CTA-pair kernels: bf16 results through shared memory + TMA stores (0: per-thread 16-byte stores)
int g_use_2cta = 1;      // 1 = CTA-pair kernel (tcgen05 cta_group::2) for the plain / row-col / SwiGLU GEMMs

// Scheduler slots of the CTA-pair kernels: {next tile, pairs done}, zero when idle (the last pair of a launch zeroes
// its slot again).  Launches on one stream follow each other and share a slot; launches on different streams may
// overlap on the GPU and get different slots.  More than kSchedSlots streams: static scheduling for the rest.
// (A CUDA graph keeps the slot of the stream it was captured on; two graphs captured on the same stream should not
// be replayed at the same time.)
constexpr int kSchedSlots = 64;
__device__ uint32_t g_sched_slots[kSchedSlots][2];
std::mutex g_sched_mu;
struct SchedKey { int dev; cudaStream_t stream; };
SchedKey g_sched_keys[kSchedSlots];
int g_sched_used = 0;
uint32_t* g_sched_base[64] = {};

uint32_t* sched_slot(cudaStream_t stream)
{
    if (!g_dynamic_tiles) return nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_sched_mu);
    if (g_sched_base[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_sched_slots) != cudaSuccess) return nullptr;
        g_sched_base[dev] = static_cast<uint32_t*>(ptr);
    }
    for (int i = 0; i < g_sched_used; ++i)
        if (g_sched_keys[i].dev == dev && g_sched_keys[i].stream == stream) return g_sched_base[dev] + 2 * i;
    if (g_sched_used == kSchedSlots) return nullptr;
    g_sched_keys[g_sched_used] = SchedKey{dev, stream};
    return g_sched_base[dev] + 2 * g_sched_used++;
}

template <int EPI, typename OutT, int BN, bool AR>
cudaError_t launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmB2, const Params& p,
                   cudaStream_t stream)
{
    auto kernel = gemm_fp8_kernel<EPI, OutT, BN, AR>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int sms = usable_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sms ? tiles : sms;
    kernel<<<grid, kBaseThreads + (AR ? kReducerThreads : 0), Cfg<BN>::kSmemBytes, stream>>>(tmA, tmB, tmB2, p);
    return cudaGetLastError();
}

template <int EPI, typename OutT, int BN>
cudaError_t launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmB2, const CUtensorMap& tmC,
                        const Params& p, cudaStream_t stream)
{
    auto kernel = gemm_fp8_2cta_kernel<EPI, OutT, BN>;
    constexpr int kPairSmemBytes = PairCfg<BN>::kSmemBytes;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int sms = usable_sms();
    if (sms <= 0) return cudaErrorInvalidDevice;
    const int tiles = p.tiles_m * p.tiles_n;
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(kBaseThreads);
    cfg.dynamicSmemBytes = kPairSmemBytes; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmB2, tmC, p);
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

// B-tile width: the persistent grid runs ceil(tiles / SMs) waves of tiles whose cost grows with
// the width; pick the width with the smaller product (224 wins when 256 leaves a ragged last wave).
int choose_bn(int M, int n_out, bool swiglu)
{
    if (g_force_bn) return g_force_bn;
    const int sms = usable_sms() > 0 ? usable_sms() : 148;
    long long best_cost = -1; int best = 256;
    for (int bn : {256, 224}) {
        const int out_cols = swiglu ? bn / 2 : bn;
        const long long tiles = static_cast<long long>((M + kBM - 1) / kBM) * ((n_out + out_cols - 1) / out_cols);
        const long long cost = ((tiles + sms - 1) / sms) * (bn + 24);     // +24: per-tile fixed cost (fill, drain)
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

}  // namespace

struct ArArgs {
    const void* const* partial_ptrs; void* const* out_ptrs; void* const* flag_ptrs;
    const void* partial_mc; void* out_mc; void* counters;
    unsigned int flag_offset_bytes, epoch; int rank, world;
};

cudaError_t gemm(const void* A, const void* B, void* C, int M, int N, int K, int epi, int out_f32, float alpha,
                 const float* row_scale, const float* col_scale, const void* B2, const float* col_scale2,
                 long long ldc, const ArArgs* ar, cudaStream_t stream, const int32_t* c_in = nullptr)
{
    if (bad_operands(A, B, C, M, N, K)) return cudaErrorInvalidValue;
    if (epi == kEpiInt32 && (!out_f32 || ar != nullptr)) return cudaErrorInvalidValue;      // 32-bit output words
    if (epi == kEpiRowCol && (row_scale == nullptr || col_scale == nullptr)) return cudaErrorInvalidValue;
    if (epi == kEpiSwiGLU &&
        (row_scale == nullptr || col_scale == nullptr || col_scale2 == nullptr || B2 == nullptr || !aligned16(B2)))
        return cudaErrorInvalidValue;
    if (ldc < N) return cudaErrorInvalidValue;

    const bool swiglu = epi == kEpiSwiGLU;
    const int bn = ar ? 256 : choose_bn(M, N, swiglu);
    const int out_cols = swiglu ? bn / 2 : bn;
    Params p{};
    p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.alpha = alpha;
    p.row_scale = row_scale; p.col_scale = col_scale; p.col_scale2 = col_scale2; p.c_in = c_in;
    p.tiles_m = (M + kBM - 1) / kBM;
    p.tiles_n = (N + out_cols - 1) / out_cols;
    p.group = 16;
    p.status = status_ptr();
    if (p.status == nullptr) return cudaErrorInvalidDevice;
    if (ar) {
        if (epi != kEpiRowCol || N % 8 != 0 || ldc != N || !aligned16(C)) return cudaErrorInvalidValue;
        if (ar->partial_ptrs == nullptr || ar->out_ptrs == nullptr || ar->flag_ptrs == nullptr || ar->counters == nullptr)
            return cudaErrorInvalidValue;
        if (ar->world < 1 || ar->world > kMaxWorld || ar->rank < 0 || ar->rank >= ar->world) return cudaErrorInvalidValue;
        if ((ar->partial_mc == nullptr) != (ar->out_mc == nullptr) || ar->flag_offset_bytes % 4 != 0) return cudaErrorInvalidValue;
        p.group = 4;                                   // 512-row groups finish (and are reduced) early
        if ((p.tiles_m + p.group - 1) / p.group > kMaxGroups) return cudaErrorInvalidValue;
        p.partial_ptrs = ar->partial_ptrs;
        p.out_ptrs = reinterpret_cast<__nv_bfloat16* const*>(ar->out_ptrs);
        p.flag_ptrs = reinterpret_cast<uint32_t* const*>(ar->flag_ptrs);
        p.partial_mc = ar->partial_mc;
        p.out_mc = static_cast<__nv_bfloat16*>(ar->out_mc);
        p.counters = static_cast<uint32_t*>(ar->counters);
        p.flag_offset_words = ar->flag_offset_bytes / 4; p.epoch = ar->epoch; p.rank = ar->rank; p.world = ar->world;
        p.reducer_stride = g_reducer_stride;
        cudaError_t e = cudaMemsetAsync(p.counters, 0, (kMaxGroups + 1) * sizeof(uint32_t), stream);
        if (e != cudaSuccess) return e;
    }

    if (g_use_2cta && !ar) {
        // CTA pairs: 256 x BN tiles (SwiGLU: BN/2 output columns); every CTA loads 128 rows of A and BN/2 rows of B
        const int sms = usable_sms() > 0 ? usable_sms() : 148;
        int pbn = 256; long long best = -1;
        for (int cand : {256, 224}) {
            if (g_force_bn && cand != g_force_bn) continue;
            const int oc = swiglu ? cand / 2 : cand;
            const long long tiles = static_cast<long long>((M + kPairBM - 1) / kPairBM) * ((N + oc - 1) / oc);
            const long long cost = ((tiles + sms / 2 - 1) / (sms / 2)) * (cand + 24);
            if (best < 0 || cost < best) { best = cost; pbn = cand; }
        }
        const int oc = swiglu ? pbn / 2 : pbn;
        CUtensorMap tA, tB, tB2;
        p.tiles_m = (M + kPairBM - 1) / kPairBM;
        p.tiles_n = (N + oc - 1) / oc;
        p.group = g_pair_group > 0 ? g_pair_group : choose_tile_group(p.tiles_m, kPairBM, static_cast<size_t>(K));
        if (!make_tmap_2d_u8(&tA, A, M, K, K, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
        if (!make_tmap_2d_u8(&tB, B, N, K, K, pbn / 2, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
        tB2 = tB;
        if (swiglu && !make_tmap_2d_u8(&tB2, B2, N, K, K, pbn / 2, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
        // bf16 results: the output as a tensor map with the epilogue's 32-row x (32- or 16-column) boxes
        CUtensorMap tC = tA;
        p.tma_store = 0;
        p.sched = sched_slot(stream);
        if (!out_f32 && g_tma_store && (ldc * 2) % 16 == 0 && aligned16(C)) {
            const uint32_t cw = (oc % 32 == 0) ? 32u : 16u;
            const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
            const uint64_t strides[1] = {static_cast<uint64_t>(ldc) * 2};
            const uint32_t box[2] = {cw, 32};
            if (encode_tiled(&tC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dims, strides, box,
                             cw == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B) != CUDA_SUCCESS)
                return cudaErrorInvalidValue;
            p.tma_store = 1;
        }
#define B200Q_PAIR(EPI, T) (pbn == 224 ? launch_pair<EPI, T, 224>(tA, tB, tB2, tC, p, stream) : launch_pair<EPI, T, 256>(tA, tB, tB2, tC, p, stream))
        switch (epi) {
        case kEpiTensor: return out_f32 ? B200Q_PAIR(kEpiTensor, float) : B200Q_PAIR(kEpiTensor, __nv_bfloat16);
        case kEpiRowCol: return out_f32 ? B200Q_PAIR(kEpiRowCol, float) : B200Q_PAIR(kEpiRowCol, __nv_bfloat16);
        case kEpiSwiGLU: return out_f32 ? cudaErrorInvalidValue : B200Q_PAIR(kEpiSwiGLU, __nv_bfloat16);
        case kEpiInt32: return B200Q_PAIR(kEpiInt32, float);        // int32 words travel as 32-bit floats' bits
        default: return cudaErrorInvalidValue;
        }
#undef B200Q_PAIR
    }

    CUtensorMap tmA, tmB, tmB2;
    const uint32_t b_rows = static_cast<uint32_t>(swiglu ? bn / 2 : bn);
    if (!make_tmap_2d_u8(&tmA, A, M, K, K, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    if (!make_tmap_2d_u8(&tmB, B, N, K, K, b_rows, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    tmB2 = tmB;
    if (swiglu && !make_tmap_2d_u8(&tmB2, B2, N, K, K, b_rows, kBK, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;

#define B200Q_LAUNCH(EPI, T, AR_) \
    (bn == 224 ? launch<EPI, T, 224, AR_>(tmA, tmB, tmB2, p, stream) : launch<EPI, T, 256, AR_>(tmA, tmB, tmB2, p, stream))
    if (ar) return out_f32 ? launch<kEpiRowCol, float, 256, true>(tmA, tmB, tmB2, p, stream)
                           : launch<kEpiRowCol, __nv_bfloat16, 256, true>(tmA, tmB, tmB2, p, stream);
    switch (epi) {
    case kEpiTensor: return out_f32 ? B200Q_LAUNCH(kEpiTensor, float, false) : B200Q_LAUNCH(kEpiTensor, __nv_bfloat16, false);
    case kEpiRowCol: return out_f32 ? B200Q_LAUNCH(kEpiRowCol, float, false) : B200Q_LAUNCH(kEpiRowCol, __nv_bfloat16, false);
    case kEpiSwiGLU:
        if (out_f32) return cudaErrorInvalidValue;
        return B200Q_LAUNCH(kEpiSwiGLU, __nv_bfloat16, false);
    case kEpiInt32: return B200Q_LAUNCH(kEpiInt32, float, false);
    default: return cudaErrorInvalidValue;
    }
#undef B200Q_LAUNCH
}

}  // namespace fp8
}  // namespace b200q

extern "C" {

int b200q_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, float scale_a, float scale_b,
                   void* stream)
{
    return b200q::fp8::gemm(A, B, C, M, N, K, b200q::fp8::kEpiTensor, 0, scale_a * scale_b, nullptr, nullptr,
                            nullptr, nullptr, N, nullptr, static_cast<cudaStream_t>(stream));
}

int b200q_gemm_i8(const void* A, const void* B, const void* C_in, void* D, int M, int N, int K, void* stream)
{
    if (D == C_in && D != nullptr) { /* in place is fine: every element is read and written by the same thread */ }
    return b200q::fp8::gemm(A, B, D, M, N, K, b200q::fp8::kEpiInt32, 1, 1.0f, nullptr, nullptr, nullptr, nullptr, N, nullptr,
                            static_cast<cudaStream_t>(stream), static_cast<const int32_t*>(C_in));
}

int b200q_gemm_fp8_rowcol(const void* A, const void* B, void* C, int M, int N, int K, const float* row_scale,
                          const float* col_scale, int out_f32, void* stream)
{
    return b200q::fp8::gemm(A, B, C, M, N, K, b200q::fp8::kEpiRowCol, out_f32, 1.0f, row_scale, col_scale, nullptr,
                            nullptr, N, nullptr, static_cast<cudaStream_t>(stream));
}

int b200q_gemm_fp8_swiglu(const void* X, const void* Wgate, const void* Wup, void* H, int M, int I, int K,
                          const float* row_scale, const float* gate_scale, const float* up_scale, void* stream)
{
    return b200q::fp8::gemm(X, Wgate, H, M, I, K, b200q::fp8::kEpiSwiGLU, 0, 1.0f, row_scale, gate_scale, Wup,
                            up_scale, I, nullptr, static_cast<cudaStream_t>(stream));
}

int b200q_gemm_fp8_rowcol_allreduce(const void* A, const void* B, void* partial_local, int M, int N, int K,
                                    const float* row_scale, const float* col_scale,
                                    const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                    void* const* flag_ptrs_dev, const void* partial_multicast, void* out_multicast,
                                    int partial_is_bf16, void* counters_local, unsigned int flag_offset_bytes,
                                    unsigned int epoch, int rank, int world, void* stream)
{
    b200q::fp8::ArArgs ar{partial_ptrs_dev, out_ptrs_dev, flag_ptrs_dev, partial_multicast, out_multicast,
                          counters_local, flag_offset_bytes, epoch, rank, world};
    return b200q::fp8::gemm(A, B, partial_local, M, N, K, b200q::fp8::kEpiRowCol, partial_is_bf16 ? 0 : 1, 1.0f, row_scale, col_scale,
                            nullptr, nullptr, N, &ar, static_cast<cudaStream_t>(stream));
}

int b200q_gemm_fp8_rowcol_allreduce_one_device(const void* const* A_host, const void* const* B_host,
                                               const float* const* row_scale_host, const float* col_scale,
                                               void* const* partial_host, void* const* counters_host,
                                               const void* const* partial_ptrs_dev, void* const* out_ptrs_dev,
                                               void* const* flag_ptrs_dev, int M, int N, int K, int partial_is_bf16,
                                               unsigned int flag_offset_bytes, unsigned int epoch, int world,
                                               int ctas_per_rank, void* stream)
{
    using namespace b200q;
    using namespace b200q::fp8;
    if (A_host == nullptr || B_host == nullptr || row_scale_host == nullptr || col_scale == nullptr || partial_host == nullptr ||
        counters_host == nullptr || partial_ptrs_dev == nullptr || out_ptrs_dev == nullptr || flag_ptrs_dev == nullptr)
        return cudaErrorInvalidValue;
    if (world < 1 || world > kOneDeviceMaxWorld || ctas_per_rank < 1 || flag_offset_bytes % 4 != 0) return cudaErrorInvalidValue;
    if (N % 8 != 0) return cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    OneDeviceArgs a{};
    a.ctas_per_rank = ctas_per_rank;
    for (int r = 0; r < world; ++r) {
        if (bad_operands(A_host[r], B_host[r], partial_host[r], M, N, K) || !aligned16(partial_host[r]) ||
            row_scale_host[r] == nullptr || counters_host[r] == nullptr)
            return cudaErrorInvalidValue;
        Params& p = a.p[r];
        p.M = M; p.N = N; p.K = K; p.C = partial_host[r]; p.ldc = N; p.alpha = 1.0f;
        p.row_scale = row_scale_host[r]; p.col_scale = col_scale; p.col_scale2 = nullptr;
        p.tiles_m = (M + kBM - 1) / kBM;
        p.tiles_n = (N + 255) / 256;
        p.group = 4;
        if ((p.tiles_m + p.group - 1) / p.group > kMaxGroups) return cudaErrorInvalidValue;
        p.status = status_ptr();
        if (p.status == nullptr) return cudaErrorInvalidDevice;
        p.partial_ptrs = partial_ptrs_dev;
        p.out_ptrs = reinterpret_cast<__nv_bfloat16* const*>(out_ptrs_dev);
        p.flag_ptrs = reinterpret_cast<uint32_t* const*>(flag_ptrs_dev);
        p.partial_mc = nullptr; p.out_mc = nullptr;
        p.counters = static_cast<uint32_t*>(counters_host[r]);
        p.flag_offset_words = flag_offset_bytes / 4; p.epoch = epoch; p.rank = r; p.world = world;
        p.reducer_stride = 1;
        cudaError_t e = cudaMemsetAsync(p.counters, 0, (kMaxGroups + 1) * sizeof(uint32_t), st);
        if (e != cudaSuccess) return e;
        if (!make_tmap_2d_u8(&a.tmA[r], A_host[r], M, K, K, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
        if (!make_tmap_2d_u8(&a.tmB[r], B_host[r], N, K, K, 256, kBK, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;
    }
    const void* fn = partial_is_bf16 ? reinterpret_cast<const void*>(gemm_fp8_allreduce_one_device_kernel<__nv_bfloat16>)
                                     : reinterpret_cast<const void*>(gemm_fp8_allreduce_one_device_kernel<float>);
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<256>::kSmemBytes);
    if (e != cudaSuccess) return e;
    void* args[1] = {&a};
    // cooperative: refused (cudaErrorCooperativeLaunchTooLarge) unless every CTA of every "rank" can be resident at once
    return cudaLaunchCooperativeKernel(fn, dim3(world * ctas_per_rank), dim3(kBaseThreads + kReducerThreads), args,
                                       Cfg<256>::kSmemBytes, st);
}

size_t b200q_fused_allreduce_flag_bytes(void)
{
    return static_cast<size_t>(b200q::fp8::kMaxGroups + 1) * b200q::fp8::kMaxWorld * sizeof(uint32_t);
}
size_t b200q_fused_allreduce_counter_bytes(void)
{
    return static_cast<size_t>(b200q::fp8::kMaxGroups + 1) * sizeof(uint32_t);
}

int b200q_fp8_set_reducer_stride(int stride)
{
    if (stride < 1 || stride > 16) return cudaErrorInvalidValue;
    b200q::fp8::g_reducer_stride = stride;
    return 0;
}

int b200q_fp8_set_sm_limit(int sms)
{
    if (sms < 0) return cudaErrorInvalidValue;
    b200q::fp8::g_sm_limit = sms;
    return 0;
}

int b200q_fp8_set_2cta(int on)
{
    b200q::fp8::g_use_2cta = on ? 1 : 0;
    return 0;
}

int b200q_fp8_set_group(int g)
{
    if (g < 0 || g > 64) return cudaErrorInvalidValue;
    b200q::fp8::g_pair_group = g;
    return 0;
}

int b200q_fp8_set_dynamic_tiles(int on)
{
    b200q::fp8::g_dynamic_tiles = on ? 1 : 0;
    return 0;
}

int b200q_fp8_set_tma_store(int on)
{
    b200q::fp8::g_tma_store = on ? 1 : 0;
    return 0;
}

int b200q_fp8_set_tile_n(int bn)
{
    if (bn != 0 && bn != 224 && bn != 256) return cudaErrorInvalidValue;
    b200q::fp8::g_force_bn = bn;
    return 0;
}

}  // extern "C"
