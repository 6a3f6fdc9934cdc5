// Shared host/device helpers of the library: status word, tensor-map encoding
// through the driver entry point, argument checks.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200q {

// Device-side status word: 0 = ok; a bounded wait that ran out stores where it gave
// up (see ptx::mbar_wait).  One word per device, defined in common.cu; kernels get
// its device address as a parameter.
uint32_t* status_ptr();   // device address for the current device (nullptr on error)

// cuTensorMapEncodeTiled obtained with cudaGetDriverEntryPoint, so the library has no
// link-time dependency on libcuda.
CUresult encode_tiled(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* gaddr,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle);

// 2-D row-major byte matrix [rows, row_bytes] with a (box_rows x box_bytes) box.
// Out-of-range box elements are read as zero.
bool make_tmap_2d_u8(CUtensorMap* map, const void* gaddr, uint64_t rows, uint64_t row_bytes,
                     uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_bytes,
                     CUtensorMapSwizzle swizzle);

int num_sms();

__host__ __device__ inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace b200q
