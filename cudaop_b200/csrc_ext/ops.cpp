// cudaop_b200._C — the torch extension in front of libb200q.so.
//
// Same conventions as the reference project's extensions (op/grouped_gemm/csrc/ops.cu:8-14,
// op/grouped_gemm/csrc/grouped_gemm.cuh:106-176, op/neuron/csrc/ops.cpp:117-139): functions take and
// return torch::Tensor, validate with TORCH_CHECK_VALUE (CUDA tensor, same device, contiguous, dtype, shape),
// run under a CUDAGuard on the inputs' device, launch on torch's current stream, allocate outputs with
// torch::empty on the inputs' device, and report failures as exceptions.  No kernel lives here: every
// function forwards raw pointers to the C ABI declared in include/b200q.h.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <c10/cuda/CUDAGuard.h>

#include <tuple>
#include <vector>

#include "../../include/b200q.h"

namespace cudaop_b200 {
namespace {

// Numbers go into error messages as ready-made strings: formatting them through an output stream (which is what the
// TORCH_CHECK macros do with non-string arguments) crashed inside the C++ runtime's locale code in this process.
std::string num(int64_t v) { return std::to_string(v); }

void check_cuda_2d(const torch::Tensor& t, const char* name, std::initializer_list<c10::ScalarType> dtypes, int64_t dim = 2)
{
    TORCH_CHECK_VALUE(t.dim() == dim, name, " must have ", num(dim), " dimensions, got ", num(t.dim()));
    TORCH_CHECK_VALUE(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK_VALUE(t.is_contiguous(), name, " must be contiguous");
    bool ok = false;
    for (auto d : dtypes) ok = ok || t.scalar_type() == d;
    TORCH_CHECK_VALUE(ok, name, " has dtype ", c10::toString(t.scalar_type()), ", which this operator does not take");
}

void same_device(std::initializer_list<const torch::Tensor*> ts)
{
    const auto dev = (*ts.begin())->device();
    for (auto* t : ts) TORCH_CHECK_VALUE(t->device() == dev, "all tensors must be on the same device");
}

void* stream_of(const torch::Tensor& t)
{
    return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

void raise_on(int code, const char* what)
{
    TORCH_CHECK(code == 0, what, " failed with cudaError ", num(code), code == 1 ? " (invalid argument)" : "");
    C10_CUDA_KERNEL_LAUNCH_CHECK();
}

constexpr auto kU8 = c10::ScalarType::Byte;
constexpr auto kE4M3 = c10::ScalarType::Float8_e4m3fn;
constexpr auto kBF16 = c10::ScalarType::BFloat16;
constexpr auto kF16 = c10::ScalarType::Half;
constexpr auto kF32 = c10::ScalarType::Float;
constexpr auto kI8 = c10::ScalarType::Char;
constexpr auto kI32 = c10::ScalarType::Int;

torch::Tensor out_like(const torch::Tensor& ref, std::vector<int64_t> shape, c10::ScalarType dt)
{
    return torch::empty(shape, ref.options().dtype(dt));
}

}  // namespace

torch::Tensor gemm_fp8(torch::Tensor a, torch::Tensor b, double scale_a, double scale_b)
{
    check_cuda_2d(a, "a", {kU8, kE4M3}); check_cuda_2d(b, "b", {kU8, kE4M3}); same_device({&a, &b});
    TORCH_CHECK_VALUE(a.size(1) == b.size(1), "inner dimensions differ: ", num(a.size(1)), " vs ", num(b.size(1)));
    const c10::cuda::CUDAGuard guard(a.device());
    auto c = out_like(a, {a.size(0), b.size(0)}, kBF16);
    raise_on(b200q_gemm_fp8(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)a.size(0), (int)b.size(0), (int)a.size(1),
                            (float)scale_a, (float)scale_b, stream_of(a)), "b200q_gemm_fp8");
    return c;
}

torch::Tensor gemm_i8(torch::Tensor a, torch::Tensor b, c10::optional<torch::Tensor> c)
{
    check_cuda_2d(a, "a", {kI8}); check_cuda_2d(b, "b", {kI8}); same_device({&a, &b});
    TORCH_CHECK_VALUE(a.size(1) == b.size(1), "inner dimensions differ: ", num(a.size(1)), " vs ", num(b.size(1)));
    const void* cin = nullptr;
    if (c.has_value()) {
        check_cuda_2d(*c, "c", {kI32}); same_device({&a, &*c});
        TORCH_CHECK_VALUE(c->size(0) == a.size(0) && c->size(1) == b.size(0), "c must be [M, N]");
        cin = c->data_ptr();
    }
    const c10::cuda::CUDAGuard guard(a.device());
    auto d = out_like(a, {a.size(0), b.size(0)}, kI32);
    raise_on(b200q_gemm_i8(a.data_ptr(), b.data_ptr(), cin, d.data_ptr(), (int)a.size(0), (int)b.size(0), (int)a.size(1), stream_of(a)),
             "b200q_gemm_i8");
    return d;
}

torch::Tensor gmm_fp8(torch::Tensor a, torch::Tensor a_scale, torch::Tensor b, torch::Tensor b_scale, torch::Tensor batch_sizes)
{
    check_cuda_2d(a, "a", {kU8, kE4M3}); check_cuda_2d(b, "b", {kU8, kE4M3}, 3);
    check_cuda_2d(a_scale, "a_scale", {kF32}, 1); check_cuda_2d(b_scale, "b_scale", {kF32}, 2);
    same_device({&a, &a_scale, &b, &b_scale});
    const int64_t T = a.size(0), K = a.size(1), E = b.size(0), N = b.size(1);
    TORCH_CHECK_VALUE(b.size(2) == K && a_scale.numel() == T && b_scale.size(0) == E && b_scale.size(1) == N, "shape mismatch");
    TORCH_CHECK_VALUE(batch_sizes.dim() == 1 && batch_sizes.numel() == E && batch_sizes.scalar_type() == c10::ScalarType::Long,
                      "batch_sizes must be a 1-D int64 tensor with one entry per expert");
    const c10::cuda::CUDAGuard guard(a.device());
    // the reference passes batch_sizes on the CPU (op/grouped_gemm/csrc/grouped_gemm.cuh:106-143); the kernel reads it on the device
    auto bs = batch_sizes.is_cuda() ? batch_sizes.contiguous() : batch_sizes.to(a.device(), /*non_blocking=*/false).contiguous();
    auto c = torch::zeros({T, N}, a.options().dtype(kBF16));
    raise_on(b200q_gmm_fp8(a.data_ptr(), a_scale.data_ptr<float>(), b.data_ptr(), b_scale.data_ptr<float>(),
                           reinterpret_cast<const long long*>(bs.data_ptr<int64_t>()), c.data_ptr(), (int)T, (int)N, (int)K, (int)E,
                           stream_of(a)), "b200q_gmm_fp8");
    return c;
}

torch::Tensor gemm_fp8_rowcol(torch::Tensor a, torch::Tensor b, torch::Tensor row_scale, torch::Tensor col_scale, bool out_f32)
{
    check_cuda_2d(a, "a", {kU8, kE4M3}); check_cuda_2d(b, "b", {kU8, kE4M3});
    check_cuda_2d(row_scale, "row_scale", {kF32}, 1); check_cuda_2d(col_scale, "col_scale", {kF32}, 1);
    same_device({&a, &b, &row_scale, &col_scale});
    TORCH_CHECK_VALUE(a.size(1) == b.size(1) && row_scale.numel() == a.size(0) && col_scale.numel() == b.size(0), "shape mismatch");
    const c10::cuda::CUDAGuard guard(a.device());
    auto c = out_like(a, {a.size(0), b.size(0)}, out_f32 ? kF32 : kBF16);
    raise_on(b200q_gemm_fp8_rowcol(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)a.size(0), (int)b.size(0), (int)a.size(1),
                                   row_scale.data_ptr<float>(), col_scale.data_ptr<float>(), out_f32 ? 1 : 0, stream_of(a)),
             "b200q_gemm_fp8_rowcol");
    return c;
}

torch::Tensor gemm_fp8_swiglu(torch::Tensor x, torch::Tensor w_gate, torch::Tensor w_up, torch::Tensor row_scale,
                              torch::Tensor gate_scale, torch::Tensor up_scale)
{
    check_cuda_2d(x, "x", {kU8, kE4M3}); check_cuda_2d(w_gate, "w_gate", {kU8, kE4M3}); check_cuda_2d(w_up, "w_up", {kU8, kE4M3});
    check_cuda_2d(row_scale, "row_scale", {kF32}, 1); check_cuda_2d(gate_scale, "gate_scale", {kF32}, 1);
    check_cuda_2d(up_scale, "up_scale", {kF32}, 1);
    same_device({&x, &w_gate, &w_up, &row_scale, &gate_scale, &up_scale});
    const int64_t M = x.size(0), K = x.size(1), I = w_gate.size(0);
    TORCH_CHECK_VALUE(w_gate.size(1) == K && w_up.size(0) == I && w_up.size(1) == K && row_scale.numel() == M &&
                gate_scale.numel() == I && up_scale.numel() == I, "shape mismatch");
    const c10::cuda::CUDAGuard guard(x.device());
    auto h = out_like(x, {M, I}, kBF16);
    raise_on(b200q_gemm_fp8_swiglu(x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), h.data_ptr(), (int)M, (int)I, (int)K,
                                   row_scale.data_ptr<float>(), gate_scale.data_ptr<float>(), up_scale.data_ptr<float>(),
                                   stream_of(x)), "b200q_gemm_fp8_swiglu");
    return h;
}

torch::Tensor gemm_w4a16(torch::Tensor x, torch::Tensor wq, torch::Tensor scales, int64_t group)
{
    check_cuda_2d(x, "x", {kBF16}); check_cuda_2d(wq, "wq", {kU8}); check_cuda_2d(scales, "scales", {kF16});
    same_device({&x, &wq, &scales});
    const int64_t M = x.size(0), K = x.size(1), N = wq.size(0);
    TORCH_CHECK_VALUE(group > 0 && wq.size(1) * 2 == K && K % group == 0 && scales.size(0) == N && scales.size(1) == K / group,
                "shape mismatch");
    const c10::cuda::CUDAGuard guard(x.device());
    auto y = out_like(x, {M, N}, kBF16);
    raise_on(b200q_gemm_w4a16(x.data_ptr(), wq.data_ptr(), scales.data_ptr(), y.data_ptr(), (int)M, (int)N, (int)K, (int)group,
                              stream_of(x)), "b200q_gemm_w4a16");
    return y;
}

torch::Tensor nvfp4_swizzle_sf(torch::Tensor sf, int64_t K)
{
    check_cuda_2d(sf, "sf", {kU8});
    TORCH_CHECK_VALUE(sf.size(1) * 16 == K && K % 64 == 0, "scales must be [rows, K/16] with K % 64 == 0");
    const c10::cuda::CUDAGuard guard(sf.device());
    auto out = out_like(sf, {(int64_t)b200q_nvfp4_sf_bytes((int)sf.size(0), (int)K)}, kU8);
    raise_on(b200q_nvfp4_swizzle_sf(sf.data_ptr(), out.data_ptr(), (int)sf.size(0), (int)K, stream_of(sf)), "b200q_nvfp4_swizzle_sf");
    return out;
}

torch::Tensor gemm_nvfp4(torch::Tensor aq, torch::Tensor sfa, torch::Tensor bq, torch::Tensor sfb, double global_a,
                         double global_b, bool blocked)
{
    check_cuda_2d(aq, "aq", {kU8}); check_cuda_2d(bq, "bq", {kU8});
    const int64_t M = aq.size(0), N = bq.size(0), K = 2 * aq.size(1);
    TORCH_CHECK_VALUE(aq.size(1) == bq.size(1) && K % 64 == 0, "shape mismatch (K must match and be a multiple of 64)");
    const c10::cuda::CUDAGuard guard(aq.device());
    auto c = out_like(aq, {M, N}, kBF16);
    if (blocked) {
        check_cuda_2d(sfa, "sfa", {kU8}, 1); check_cuda_2d(sfb, "sfb", {kU8}, 1);
        same_device({&aq, &sfa, &bq, &sfb});
        TORCH_CHECK_VALUE(sfa.numel() == (int64_t)b200q_nvfp4_sf_bytes((int)M, (int)K) && sfb.numel() == (int64_t)b200q_nvfp4_sf_bytes((int)N, (int)K),
                    "blocked scale arrays have the wrong size");
        raise_on(b200q_gemm_nvfp4_blocked(aq.data_ptr(), sfa.data_ptr(), bq.data_ptr(), sfb.data_ptr(), c.data_ptr(), (int)M, (int)N,
                                          (int)K, (float)global_a, (float)global_b, stream_of(aq)), "b200q_gemm_nvfp4_blocked");
        return c;
    }
    check_cuda_2d(sfa, "sfa", {kU8}); check_cuda_2d(sfb, "sfb", {kU8});
    same_device({&aq, &sfa, &bq, &sfb});
    TORCH_CHECK_VALUE(sfa.size(0) == M && sfa.size(1) == K / 16 && sfb.size(0) == N && sfb.size(1) == K / 16, "shape mismatch");
    auto ws = out_like(aq, {(int64_t)b200q_gemm_nvfp4_workspace_bytes((int)M, (int)N, (int)K)}, kU8);
    raise_on(b200q_gemm_nvfp4(aq.data_ptr(), sfa.data_ptr(), bq.data_ptr(), sfb.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K,
                              (float)global_a, (float)global_b, ws.data_ptr(), stream_of(aq)), "b200q_gemm_nvfp4");
    return c;
}

torch::Tensor mxfp8_swizzle_sf(torch::Tensor sf, int64_t K)
{
    check_cuda_2d(sf, "sf", {kU8});
    TORCH_CHECK_VALUE(sf.size(1) * 32 == K, "scales must be [rows, K/32]");
    const c10::cuda::CUDAGuard guard(sf.device());
    auto out = out_like(sf, {(int64_t)b200q_mxfp8_sf_bytes((int)sf.size(0), (int)K)}, kU8);
    raise_on(b200q_mxfp8_swizzle_sf(sf.data_ptr(), out.data_ptr(), (int)sf.size(0), (int)K, stream_of(sf)), "b200q_mxfp8_swizzle_sf");
    return out;
}

torch::Tensor gemm_mxfp8(torch::Tensor a, torch::Tensor sfa, torch::Tensor b, torch::Tensor sfb, bool blocked)
{
    check_cuda_2d(a, "a", {kU8, kE4M3}); check_cuda_2d(b, "b", {kU8, kE4M3});
    const int64_t M = a.size(0), N = b.size(0), K = a.size(1);
    TORCH_CHECK_VALUE(b.size(1) == K && K % 32 == 0, "shape mismatch (K must match and be a multiple of 32)");
    const c10::cuda::CUDAGuard guard(a.device());
    auto c = out_like(a, {M, N}, kBF16);
    if (blocked) {
        check_cuda_2d(sfa, "sfa", {kU8}, 1); check_cuda_2d(sfb, "sfb", {kU8}, 1);
        same_device({&a, &sfa, &b, &sfb});
        TORCH_CHECK_VALUE(sfa.numel() == (int64_t)b200q_mxfp8_sf_bytes((int)M, (int)K) && sfb.numel() == (int64_t)b200q_mxfp8_sf_bytes((int)N, (int)K),
                          "blocked scale arrays have the wrong size");
        raise_on(b200q_gemm_mxfp8_blocked(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K,
                                          stream_of(a)), "b200q_gemm_mxfp8_blocked");
        return c;
    }
    check_cuda_2d(sfa, "sfa", {kU8}); check_cuda_2d(sfb, "sfb", {kU8});
    same_device({&a, &sfa, &b, &sfb});
    TORCH_CHECK_VALUE(sfa.size(0) == M && sfa.size(1) == K / 32 && sfb.size(0) == N && sfb.size(1) == K / 32, "shape mismatch");
    auto ws = out_like(a, {(int64_t)b200q_gemm_mxfp8_workspace_bytes((int)M, (int)N, (int)K)}, kU8);
    raise_on(b200q_gemm_mxfp8(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K,
                              ws.data_ptr(), stream_of(a)), "b200q_gemm_mxfp8");
    return c;
}

torch::Tensor gemm_sparse_fp8(torch::Tensor a_comp, torch::Tensor a_meta, torch::Tensor b, double scale_a, double scale_b)
{
    check_cuda_2d(a_comp, "a_comp", {kU8, kE4M3}); check_cuda_2d(a_meta, "a_meta", {kU8}); check_cuda_2d(b, "b", {kU8, kE4M3});
    same_device({&a_comp, &a_meta, &b});
    const int64_t M = a_comp.size(0), N = b.size(0), K = b.size(1);
    TORCH_CHECK_VALUE(a_comp.size(1) * 2 == K && a_meta.size(0) == M && a_meta.size(1) == K / 8, "shape mismatch");
    const c10::cuda::CUDAGuard guard(b.device());
    auto c = out_like(b, {M, N}, kBF16);
    raise_on(b200q_gemm_sp24_fp8(a_comp.data_ptr(), a_meta.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K,
                                 (float)scale_a, (float)scale_b, stream_of(b)), "b200q_gemm_sp24_fp8");
    return c;
}

std::tuple<torch::Tensor, torch::Tensor> quant_rows_e4m3(torch::Tensor x)
{
    check_cuda_2d(x, "x", {kBF16});
    const c10::cuda::CUDAGuard guard(x.device());
    auto q = out_like(x, {x.size(0), x.size(1)}, kU8);
    auto s = out_like(x, {x.size(0)}, kF32);
    raise_on(b200q_quant_rows_e4m3(x.data_ptr(), q.data_ptr(), s.data_ptr<float>(), (int)x.size(0), (int)x.size(1), stream_of(x)),
             "b200q_quant_rows_e4m3");
    return {q, s};
}

std::tuple<torch::Tensor, torch::Tensor> quant_rows_nvfp4(torch::Tensor x, double global_scale)
{
    check_cuda_2d(x, "x", {kBF16});
    TORCH_CHECK_VALUE(x.size(1) % 64 == 0, "the row length must be a multiple of 64");
    TORCH_CHECK_VALUE(global_scale > 0.0, "global_scale must be positive");
    const c10::cuda::CUDAGuard guard(x.device());
    auto q = out_like(x, {x.size(0), x.size(1) / 2}, kU8);
    auto sf = out_like(x, {(int64_t)b200q_nvfp4_sf_bytes((int)x.size(0), (int)x.size(1))}, kU8);
    raise_on(b200q_quant_rows_nvfp4(x.data_ptr(), q.data_ptr(), sf.data_ptr(), (int)x.size(0), (int)x.size(1), (float)global_scale,
                                    stream_of(x)), "b200q_quant_rows_nvfp4");
    return {q, sf};
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.def("gemm_fp8", &gemm_fp8, "FP8 E4M3 GEMM, per-tensor scales, bf16 out");
    m.def("gemm_i8", &gemm_i8, "exact INT8 GEMM with int32 accumulation", pybind11::arg("a"), pybind11::arg("b"), pybind11::arg("c") = pybind11::none());
    m.def("gmm_fp8", &gmm_fp8, "grouped (ragged-M) FP8 GEMM");
    m.def("gemm_fp8_rowcol", &gemm_fp8_rowcol, "FP8 E4M3 GEMM, per-row x per-column scales");
    m.def("gemm_fp8_swiglu", &gemm_fp8_swiglu, "fused gate/up projection + SwiGLU on FP8 operands");
    m.def("gemm_w4a16", &gemm_w4a16, "INT4 weight-only GEMM, bf16 activations");
    m.def("nvfp4_swizzle_sf", &nvfp4_swizzle_sf, "row-major UE4M3 scales -> blocked layout");
    m.def("gemm_nvfp4", &gemm_nvfp4, "NVFP4 block-scaled GEMM");
    m.def("mxfp8_swizzle_sf", &mxfp8_swizzle_sf, "row-major UE8M0 scales -> blocked layout");
    m.def("gemm_mxfp8", &gemm_mxfp8, "MXFP8 block-scaled GEMM");
    m.def("gemm_sparse_fp8", &gemm_sparse_fp8, "2:4-sparse FP8 GEMM");
    m.def("quant_rows_e4m3", &quant_rows_e4m3, "bf16 rows -> E4M3 + per-row fp32 scale");
    m.def("quant_rows_nvfp4", &quant_rows_nvfp4, "bf16 rows -> packed E2M1 + blocked UE4M3 scales");
}

}  // namespace cudaop_b200
