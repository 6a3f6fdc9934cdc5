// Status word, tensor-map encoding and device queries shared by all operators.
#include "common.cuh"
#include "ptx.cuh"
#include "../../include/b200q.h"

#include <mutex>

namespace b200q {

// word 0: status; words 2-3 / 4-5: wait limits in ns (inside one GPU / across ranks), see ptx.cuh
__device__ __align__(16) uint32_t g_status_block[ptx::kStatusBlockWords] = {
    0u, 0u,
    static_cast<uint32_t>(ptx::kDefaultLocalWaitNs & 0xFFFFFFFFull), static_cast<uint32_t>(ptx::kDefaultLocalWaitNs >> 32),
    static_cast<uint32_t>(ptx::kDefaultPeerWaitNs & 0xFFFFFFFFull), static_cast<uint32_t>(ptx::kDefaultPeerWaitNs >> 32),
    0u, 0u};

namespace {
constexpr int kMaxDevices = 64;
uint32_t* g_status_addr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
std::mutex g_mu;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
}  // namespace

uint32_t* status_ptr()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_status_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_block) != cudaSuccess) return nullptr;
        g_status_addr[dev] = static_cast<uint32_t*>(p);
    }
    return g_status_addr[dev];
}

int num_sms()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

CUresult encode_tiled(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* gaddr,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle)
{
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (g_encode == nullptr) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
                fn == nullptr || q != cudaDriverEntryPointSuccess)
                return CUDA_ERROR_NOT_SUPPORTED;
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        }
    }
    cuuint64_t d[5]; cuuint64_t s[5]; cuuint32_t b[5]; cuuint32_t e[5];
    for (uint32_t i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; e[i] = 1; }
    for (uint32_t i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
    return g_encode(map, dtype, rank, const_cast<void*>(gaddr), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

bool make_tmap_2d_u8(CUtensorMap* map, const void* gaddr, uint64_t rows, uint64_t row_bytes,
                     uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_bytes,
                     CUtensorMapSwizzle swizzle)
{
    const uint64_t dims[2] = {row_bytes, rows};
    const uint64_t strides[1] = {row_stride_bytes};
    const uint32_t box[2] = {box_bytes, box_rows};
    return encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, gaddr, dims, strides, box, swizzle) == CUDA_SUCCESS;
}

}  // namespace b200q

extern "C" int b200q_status(unsigned int* host_out, int clear)
{
    using namespace b200q;
    if (host_out == nullptr) return cudaErrorInvalidValue;
    uint32_t* p = status_ptr();
    if (p == nullptr) return cudaErrorInvalidDevice;
    cudaError_t e = cudaMemcpy(host_out, p, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    if (clear) e = cudaMemset(p, 0, sizeof(uint32_t));
    return e;
}

extern "C" int b200q_set_wait_limit_ms(int kind, int ms)
{
    using namespace b200q;
    if ((kind != 0 && kind != 1) || ms < 1 || ms > 600000) return cudaErrorInvalidValue;
    uint32_t* p = status_ptr();
    if (p == nullptr) return cudaErrorInvalidDevice;
    const unsigned long long ns = static_cast<unsigned long long>(ms) * 1000000ull;
    return cudaMemcpy(p + (kind == 0 ? 2 : 4), &ns, sizeof(ns), cudaMemcpyHostToDevice);
}
