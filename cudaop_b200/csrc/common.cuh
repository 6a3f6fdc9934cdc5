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

// Tile order of the persistent CTA-pair GEMMs: `group` tile rows walk the N tiles together, so the A rows of a group
// stay in L2 while B streams past them once per group.  Measured (8192^3 FP8 and NVFP4, the MLP shapes): the best
// group is the largest power of two whose A rows fit in about 60 MB of the 126 MB L2.
inline int choose_tile_group(int tiles_m, size_t rows_per_tile, size_t row_bytes)
{
    const size_t budget = 60u << 20;
    int g = 1;
    while (g < tiles_m && g * 2 <= 64 && static_cast<size_t>(g * 2) * rows_per_tile * row_bytes <= budget) g *= 2;
    return g;
}

__host__ __device__ inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace b200q
