// Unmangled entry to the reference's own CPU GEMM (op/cpu/cpu_ops.h:34-39), so a
// test can load the compiled reference with ctypes.  Holds no arithmetic.
#include "cpu_ops.h"
extern "C" void cudaop_ref_gemm_mma_cpu(const float* A, const float* B, float* C, int M, int N, int K)
{
    gemm_mma_cpu(A, B, C, M, N, K);
}
