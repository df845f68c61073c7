// Python operator surface `my_int4._C`: the same 16 callables, argument names, shapes,
// dtypes and error type (RuntimeError) as the reference's csrc/bindings.cpp:28-68, each a
// thin wrapper over the C ABI of include/wush_int4.h.  The wrappers validate, allocate the
// outputs (and scratch) through torch's caching allocator, pick the current stream and
// launch -- no host synchronisation, so every op can be captured in a CUDA Graph.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "../../include/wush_int4.h"

namespace {

void check_status(int status, const char* op)
{
    TORCH_CHECK(status == WUSH_OK, op, ": ", wush_last_error(), " (status ", status, ")");
}

cudaStream_t stream_of(const torch::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

void check_bf16_cuda(const torch::Tensor& t, const char* name)
{
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
    TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bf16");
}

std::vector<int64_t> with_last(const torch::Tensor& t, int64_t last)
{
    std::vector<int64_t> s = t.sizes().vec();
    s.back() = last;
    return s;
}

// ---- a1 -------------------------------------------------------------------------------
std::vector<torch::Tensor> quant_int4(torch::Tensor x)
{
    check_bf16_cuda(x, "x");
    TORCH_CHECK(x.dim() >= 1 && x.size(-1) % 32 == 0, "last dim must be multiple of 32");
    const at::cuda::OptionalCUDAGuard guard(x.device());
    const int64_t K = x.size(-1);
    auto q = torch::empty(with_last(x, K / 2), x.options().dtype(torch::kUInt8));
    auto s = torch::empty(with_last(x, K / 32), x.options());
    check_status(wush_quant_int4(x.data_ptr(), x.numel() / 32, q.data_ptr<uint8_t>(), s.data_ptr(), stream_of(x)),
                 "quant_int4");
    return {q, s};
}

// ---- a4..a7 ---------------------------------------------------------------------------
std::vector<torch::Tensor> fused_tq(torch::Tensor x, torch::Tensor t, int variant, const char* op)
{
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && t.is_cuda() && t.is_contiguous(),
                "x/t must be contiguous CUDA tensors");
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && t.scalar_type() == torch::kBFloat16, "x/t must be bf16");
    TORCH_CHECK(x.dim() >= 1 && t.dim() == 3, "T must be (K/32, 32, 32)");
    const int64_t K = x.size(-1), C = K / 32;
    TORCH_CHECK(K % 32 == 0 && t.size(0) == C && t.size(1) == 32 && t.size(2) == 32, "T must be (K/32, 32, 32)");
    TORCH_CHECK(x.device() == t.device(), "x and t must be on the same device");
    const at::cuda::OptionalCUDAGuard guard(x.device());
    const int64_t rows = K ? x.numel() / K : 0;
    auto q = torch::empty(with_last(x, K / 2), x.options().dtype(torch::kUInt8));
    auto s = torch::empty(with_last(x, C), x.options());
    check_status(wush_fused_transform_quant_int4(x.data_ptr(), t.data_ptr(), rows, K, variant, q.data_ptr<uint8_t>(),
                                                 s.data_ptr(), stream_of(x)),
                 op);
    return {q, s};
}
std::vector<torch::Tensor> fused_transform_quant_int4(torch::Tensor x, torch::Tensor t)
{
    return fused_tq(x, t, WUSH_TQ_EXACT, "fused_transform_quant_int4");
}
// Addition to the reference surface: SiLU(gate) * up -> bf16 -> transform -> quantise in one pass
// over the fp16 output of a fused gate+up projection (gate half first).
std::vector<torch::Tensor> fused_silu_mul_transform_quant_int4(torch::Tensor gate_up, torch::Tensor t)
{
    TORCH_CHECK(gate_up.is_cuda() && gate_up.is_contiguous() && t.is_cuda() && t.is_contiguous(),
                "gate_up/t must be contiguous CUDA tensors");
    TORCH_CHECK(gate_up.scalar_type() == torch::kHalf && t.scalar_type() == torch::kBFloat16,
                "gate_up must be fp16, t bf16");
    TORCH_CHECK(gate_up.dim() >= 1 && t.dim() == 3 && gate_up.size(-1) % 64 == 0, "gate_up must be (..., 2K), K % 32 == 0");
    const int64_t K = gate_up.size(-1) / 2, C = K / 32;
    TORCH_CHECK(t.size(0) == C && t.size(1) == 32 && t.size(2) == 32, "T must be (K/32, 32, 32)");
    TORCH_CHECK(gate_up.device() == t.device(), "gate_up and t must be on the same device");
    const at::cuda::OptionalCUDAGuard guard(gate_up.device());
    const int64_t rows = gate_up.numel() / (2 * K);
    auto q = torch::empty(with_last(gate_up, K / 2), gate_up.options().dtype(torch::kUInt8));
    auto s = torch::empty(with_last(gate_up, C), gate_up.options().dtype(torch::kBFloat16));
    check_status(wush_fused_silu_mul_transform_quant_int4(gate_up.data_ptr(), t.data_ptr(), rows, K, q.data_ptr<uint8_t>(),
                                                          s.data_ptr(), stream_of(gate_up)),
                 "fused_silu_mul_transform_quant_int4");
    return {q, s};
}
std::vector<torch::Tensor> fused_transform_quant_int4_wmma(torch::Tensor x, torch::Tensor t)
{
    return fused_tq(x, t, WUSH_TQ_FAST, "fused_transform_quant_int4_wmma");
}
std::vector<torch::Tensor> fused_transform_quant_int4_v3(torch::Tensor x, torch::Tensor t)
{
    return fused_tq(x, t, WUSH_TQ_FAST, "fused_transform_quant_int4_v3");
}
std::vector<torch::Tensor> fused_transform_quant_int4_smallm(torch::Tensor x, torch::Tensor t)
{
    TORCH_CHECK(x.numel() >= 1, "rows must be >= 1");
    return fused_tq(x, t, WUSH_TQ_FAST, "fused_transform_quant_int4_smallm");
}

// ---- a8..a10 --------------------------------------------------------------------------
struct GemmArgs {
    int64_t M, N, K;
};

GemmArgs check_gemm(const torch::Tensor& xq, const torch::Tensor& xs, const torch::Tensor& wq, const torch::Tensor& ws)
{
    TORCH_CHECK(xq.is_cuda() && wq.is_cuda() && xs.is_cuda() && ws.is_cuda(), "tensors must be CUDA");
    TORCH_CHECK(xq.scalar_type() == torch::kUInt8 && wq.scalar_type() == torch::kUInt8, "packed tensors must be uint8");
    TORCH_CHECK(xs.scalar_type() == torch::kBFloat16 && ws.scalar_type() == torch::kBFloat16, "scales must be bf16");
    TORCH_CHECK(xq.is_contiguous() && xs.is_contiguous() && wq.is_contiguous() && ws.is_contiguous(),
                "tensors must be contiguous");
    TORCH_CHECK(wq.dim() == 2, "w must be 2D (N, K/2)");
    TORCH_CHECK(xq.dim() >= 1 && xs.dim() >= 1 && ws.dim() >= 1, "tensors must have at least one dimension");
    const int64_t K2 = xq.size(-1), K = K2 * 2, G = K / 32;
    TORCH_CHECK(K % 32 == 0, "K must be a multiple of 32");
    TORCH_CHECK(wq.size(1) == K2 && ws.size(-1) == G && xs.size(-1) == G, "K mismatch between x/w tensors");
    const int64_t M = K2 ? xq.numel() / K2 : 0, N = wq.size(0);
    TORCH_CHECK(xs.numel() == M * G && ws.numel() == N * G, "scale tensors do not match the packed tensors");
    TORCH_CHECK(xq.device() == wq.device() && xq.device() == xs.device() && xq.device() == ws.device(),
                "tensors must be on the same device");
    return {M, N, K};
}

torch::Tensor run_gemm(const torch::Tensor& xq, const torch::Tensor& xs, const torch::Tensor& wq,
                       const torch::Tensor& ws, const GemmArgs& a, std::vector<int64_t> yshape, int variant,
                       const char* op)
{
    const at::cuda::OptionalCUDAGuard guard(xq.device());
    auto y = torch::empty(yshape, xq.options().dtype(torch::kHalf));
    const size_t wbytes = wush_w4a4_gemm_workspace_bytes(a.M, a.N, a.K, variant);
    torch::Tensor work;
    if (wbytes) work = torch::empty({(int64_t)wbytes}, xq.options().dtype(torch::kUInt8));
    check_status(wush_w4a4_gemm(xq.data_ptr<uint8_t>(), xs.data_ptr(), wq.data_ptr<uint8_t>(), ws.data_ptr(), a.M, a.N,
                                a.K, y.data_ptr(), variant, wbytes ? work.data_ptr() : nullptr, wbytes, stream_of(xq)),
                 op);
    return y;
}

// v0 keeps the leading dimensions of x (reference csrc/gemm_int4.cu:128-129).
torch::Tensor w4a4_gemm(torch::Tensor xq, torch::Tensor xs, torch::Tensor wq, torch::Tensor ws)
{
    auto a = check_gemm(xq, xs, wq, ws);
    return run_gemm(xq, xs, wq, ws, a, with_last(xq, a.N), WUSH_GEMM_AUTO, "w4a4_gemm");
}
// v1 / v2 / s4 return a 2-D (M, N) tensor (reference csrc/gemm_wmma.cu:171, csrc/gemm_s4.cu:378).
torch::Tensor w4a4_gemm_v1(torch::Tensor xq, torch::Tensor xs, torch::Tensor wq, torch::Tensor ws)
{
    auto a = check_gemm(xq, xs, wq, ws);
    return run_gemm(xq, xs, wq, ws, a, {a.M, a.N}, WUSH_GEMM_AUTO, "w4a4_gemm_v1");
}
torch::Tensor w4a4_gemm_v2(torch::Tensor xq, torch::Tensor xs, torch::Tensor wq, torch::Tensor ws)
{
    auto a = check_gemm(xq, xs, wq, ws);
    TORCH_CHECK(a.K % 64 == 0, "K must be multiple of 64");
    return run_gemm(xq, xs, wq, ws, a, {a.M, a.N}, WUSH_GEMM_AUTO, "w4a4_gemm_v2");
}
torch::Tensor w4a4_gemm_s4(torch::Tensor xq, torch::Tensor xs, torch::Tensor wq, torch::Tensor ws)
{
    auto a = check_gemm(xq, xs, wq, ws);
    TORCH_CHECK(a.K % 64 == 0, "K must be multiple of 64");
    return run_gemm(xq, xs, wq, ws, a, {a.M, a.N}, WUSH_GEMM_AUTO, "w4a4_gemm_s4");
}

// ---- a9 -------------------------------------------------------------------------------
torch::Tensor w4a4_gemv(torch::Tensor xq, torch::Tensor xs, torch::Tensor wq, torch::Tensor ws)
{
    TORCH_CHECK(xq.dim() >= 1 && xq.dim() <= 2 && xq.numel() == xq.size(-1), "gemv expects a single row");
    auto a = check_gemm(xq, xs, wq, ws);
    return run_gemm(xq, xs, wq, ws, a, {a.N}, WUSH_GEMM_AUTO, "w4a4_gemv");
}
// The reference accepts 1 <= M <= 8 (csrc/gemv_int4.cu:160); this build takes up to 32 rows.
torch::Tensor w4a4_gemv_multi(torch::Tensor xq, torch::Tensor xs, torch::Tensor wq, torch::Tensor ws)
{
    auto a = check_gemm(xq, xs, wq, ws);
    TORCH_CHECK(a.M >= 1 && a.M <= 32, "gemv_multi expects 1<=M<=32");
    return run_gemm(xq, xs, wq, ws, a, {a.M, a.N}, WUSH_GEMM_AUTO, "w4a4_gemv_multi");
}

// ---- a11 ------------------------------------------------------------------------------
torch::Tensor s4_atom_selftest(torch::Tensor a, torch::Tensor b)
{
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.is_contiguous() && b.is_contiguous(), "a/b must be contiguous CUDA tensors");
    TORCH_CHECK(a.scalar_type() == torch::kInt8 && b.scalar_type() == torch::kInt8, "a/b must be int8");
    TORCH_CHECK(a.numel() == 8 * 32 && b.numel() == 32 * 8, "a must be (8,32) and b (32,8)");
    const at::cuda::OptionalCUDAGuard guard(a.device());
    auto c = torch::zeros({8, 8}, a.options().dtype(torch::kInt32));
    check_status(wush_i8_atom_selftest(a.data_ptr<int8_t>(), b.data_ptr<int8_t>(), c.data_ptr<int32_t>(), stream_of(a)),
                 "s4_atom_selftest");
    return c;
}

// Exact per-group partial sums P[m][n][g] from the tensor-core path (test-only addition).
torch::Tensor w4a4_group_partials(torch::Tensor xq, torch::Tensor wq)
{
    TORCH_CHECK(xq.is_cuda() && wq.is_cuda() && xq.is_contiguous() && wq.is_contiguous(), "tensors must be contiguous CUDA");
    TORCH_CHECK(xq.scalar_type() == torch::kUInt8 && wq.scalar_type() == torch::kUInt8, "packed tensors must be uint8");
    TORCH_CHECK(wq.dim() == 2 && xq.dim() >= 1 && xq.size(-1) == wq.size(1), "K mismatch");
    const int64_t K2 = wq.size(1), K = K2 * 2, M = xq.numel() / K2, N = wq.size(0);
    TORCH_CHECK(K % 32 == 0, "K must be a multiple of 32");
    const at::cuda::OptionalCUDAGuard guard(xq.device());
    auto P = torch::empty({M, N, K / 32}, xq.options().dtype(torch::kInt32));
    check_status(wush_group_partials(xq.data_ptr<uint8_t>(), wq.data_ptr<uint8_t>(), M, N, K, P.data_ptr<int32_t>(),
                                     stream_of(xq)),
                 "w4a4_group_partials");
    return P;
}

// ---- per-tensor route -----------------------------------------------------------------
torch::Tensor quant_int4_tensor_scale(torch::Tensor x, double scale)
{
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == torch::kBFloat16, "x must be contiguous CUDA bf16");
    TORCH_CHECK(x.numel() % 32 == 0, "numel must be multiple of 32");
    const at::cuda::OptionalCUDAGuard guard(x.device());
    auto q = torch::empty({x.numel() / 2}, x.options().dtype(torch::kUInt8));
    const float inv = (float)(1.0 / scale);              // same rounding as the reference host code
    check_status(wush_quant_int4_tensor_scale(x.data_ptr(), x.numel(), inv, nullptr, q.data_ptr<uint8_t>(), stream_of(x)),
                 "quant_int4_tensor_scale");
    return q;
}
torch::Tensor quant_int4_tensor_scale_dev(torch::Tensor x, torch::Tensor inv_scale)
{
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == torch::kBFloat16, "x must be contiguous CUDA bf16");
    TORCH_CHECK(x.numel() % 32 == 0, "numel must be multiple of 32");
    TORCH_CHECK(inv_scale.is_cuda() && inv_scale.scalar_type() == torch::kFloat32 && inv_scale.is_contiguous() &&
                    inv_scale.numel() == 1,
                "inv_scale must be 1-elem contiguous fp32 CUDA tensor");
    const at::cuda::OptionalCUDAGuard guard(x.device());
    auto q = torch::empty({x.numel() / 2}, x.options().dtype(torch::kUInt8));
    check_status(wush_quant_int4_tensor_scale(x.data_ptr(), x.numel(), 0.f, inv_scale.data_ptr<float>(),
                                              q.data_ptr<uint8_t>(), stream_of(x)),
                 "quant_int4_tensor_scale_dev");
    return q;
}

torch::Tensor gemm_ts(torch::Tensor xq, torch::Tensor wq, float alpha, const float* alpha_dev, const char* op)
{
    TORCH_CHECK(xq.is_cuda() && wq.is_cuda(), "tensors must be CUDA");
    TORCH_CHECK(xq.scalar_type() == torch::kUInt8 && wq.scalar_type() == torch::kUInt8, "packed tensors must be uint8");
    TORCH_CHECK(xq.is_contiguous() && wq.is_contiguous(), "tensors must be contiguous");
    TORCH_CHECK(wq.dim() == 2, "w must be 2D (N, K/2)");
    const int64_t K2 = wq.size(1);                       // K comes from wq; xq may be flat
    TORCH_CHECK(K2 > 0 && (K2 * 2) % 32 == 0, "K must be a multiple of 32");
    const int64_t M = xq.numel() / K2, N = wq.size(0);
    TORCH_CHECK(M * K2 == xq.numel(), "xq numel must equal M*K/2 (K from wq)");
    const at::cuda::OptionalCUDAGuard guard(xq.device());
    auto y = torch::empty({M, N}, xq.options().dtype(torch::kHalf));
    const size_t nbytes = wush_w4a4_gemm_tensor_scale_workspace_bytes(M, N, K2 * 2);
    torch::Tensor work;
    if (nbytes) work = torch::empty({(int64_t)nbytes}, xq.options());
    check_status(wush_w4a4_gemm_tensor_scale_ws(xq.data_ptr<uint8_t>(), wq.data_ptr<uint8_t>(), M, N, K2 * 2, alpha, alpha_dev,
                                                y.data_ptr(), nbytes ? work.data_ptr() : nullptr, nbytes, stream_of(xq)),
                 op);
    return y;
}
torch::Tensor w4a4_gemm_cutlass(torch::Tensor xq, torch::Tensor wq, double alpha)
{
    return gemm_ts(xq, wq, (float)alpha, nullptr, "w4a4_gemm_cutlass");
}
torch::Tensor w4a4_gemm_cutlass_dev(torch::Tensor xq, torch::Tensor wq, torch::Tensor alpha)
{
    TORCH_CHECK(alpha.is_cuda() && alpha.scalar_type() == torch::kFloat32 && alpha.is_contiguous() && alpha.numel() == 1,
                "alpha must be 1-elem contiguous fp32 CUDA tensor");
    return gemm_ts(xq, wq, 0.f, alpha.data_ptr<float>(), "w4a4_gemm_cutlass_dev");
}

void init() { check_status(wush_init(), "init"); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.def("quant_int4_tensor_scale", &quant_int4_tensor_scale, "Per-tensor INT4 quantise, host scale", py::arg("x"),
          py::arg("scale"));
    m.def("quant_int4_tensor_scale_dev", &quant_int4_tensor_scale_dev,
          "Per-tensor INT4 quantise, inv_scale read from a 1-element fp32 device tensor (graph-safe)", py::arg("x"),
          py::arg("inv_scale"));
    m.def("quant_int4", &quant_int4, "sigma-clip INT4 group quantise (G=32, bf16 scales)", py::arg("x"));
    m.def("w4a4_gemm", &w4a4_gemm, "W4A4 group-scaled product, keeps leading dims", py::arg("xq"), py::arg("xs"),
          py::arg("wq"), py::arg("ws"));
    m.def("w4a4_gemm_v1", &w4a4_gemm_v1, "W4A4 group-scaled product (alias of the current kernels)", py::arg("xq"),
          py::arg("xs"), py::arg("wq"), py::arg("ws"));
    m.def("w4a4_gemm_cutlass", &w4a4_gemm_cutlass, "W4A4 product with one scalar scale", py::arg("xq"), py::arg("wq"),
          py::arg("alpha"));
    m.def("w4a4_gemm_cutlass_dev", &w4a4_gemm_cutlass_dev,
          "W4A4 product with one scalar scale read from a 1-element fp32 device tensor (graph-safe)", py::arg("xq"),
          py::arg("wq"), py::arg("alpha"));
    m.def("w4a4_gemm_s4", &w4a4_gemm_s4, "W4A4 group-scaled product (main entry)", py::arg("xq"), py::arg("xs"),
          py::arg("wq"), py::arg("ws"));
    m.def("s4_atom_selftest", &s4_atom_selftest, "(8,32)x(32,8) int8 -> int32 through one tensor-core atom");
    m.def("w4a4_gemv", &w4a4_gemv, "W4A4 GEMV (one activation row)", py::arg("xq"), py::arg("xs"), py::arg("wq"),
          py::arg("ws"));
    m.def("w4a4_gemv_multi", &w4a4_gemv_multi, "W4A4 GEMV, 1<=M<=32", py::arg("xq"), py::arg("xs"), py::arg("wq"),
          py::arg("ws"));
    m.def("fused_transform_quant_int4_v3", &fused_transform_quant_int4_v3, "Fused WUSH transform + INT4 quantise (fast)",
          py::arg("x"), py::arg("t"));
    m.def("fused_transform_quant_int4_smallm", &fused_transform_quant_int4_smallm,
          "Fused WUSH transform + INT4 quantise (decode shapes)", py::arg("x"), py::arg("t"));
    m.def("fused_silu_mul_transform_quant_int4", &fused_silu_mul_transform_quant_int4,
          "SiLU(gate) * up -> bf16 -> WUSH transform + INT4 quantise, from the fp16 (..., 2K) gate+up output",
          py::arg("gate_up"), py::arg("t"));
    m.def("fused_transform_quant_int4", &fused_transform_quant_int4,
          "Fused WUSH transform + INT4 quantise (bit-exact serial arithmetic)", py::arg("x"), py::arg("t"));
    m.def("w4a4_gemm_v2", &w4a4_gemm_v2, "W4A4 group-scaled product (alias of the current kernels)", py::arg("xq"),
          py::arg("xs"), py::arg("wq"), py::arg("ws"));
    m.def("fused_transform_quant_int4_wmma", &fused_transform_quant_int4_wmma,
          "Fused WUSH transform + INT4 quantise (tensor-core transform)", py::arg("x"), py::arg("t"));
    // additions of this build
    m.def("w4a4_group_partials", &w4a4_group_partials, "exact int32 partial sums per group (test op)", py::arg("xq"),
          py::arg("wq"));
    m.def("init", &init, "one-time per-device set-up; call before CUDA Graph capture");
}
