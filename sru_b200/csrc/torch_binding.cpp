// Torch operator binding: registers the reference's eight operator names in the
// `sru_cuda` namespace with unchanged schemas (sru/csrc/sru_cuda_impl.cpp:177-518,
// registration :531-546) on top of the C ABI of include/sru_b200.h.  TorchScript programs
// and C++ applications that reach the kernels by operator name keep working against this
// library.  Differences inside the boundary: launches go to the current CUDA stream, outputs
// are allocated uninitialised (the kernels write every element), failures raise c10::Error.
//
// The backward operators return grad_weight_c / grad_bias already reduced over the batch,
// shaped (2, 1, D): the reference's Python caller applies `.sum(1).view(-1)` to a
// (2, batch, D) tensor of partials (sru/cuda_functional.py:258-260) and gets the same result.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include <algorithm>
#include <vector>

#include "../../include/sru_b200.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<at::Tensor>;

int dtype_code(at::ScalarType t) {
    switch (t) {
        case at::kFloat: return SRU_F32;
        case at::kHalf: return SRU_F16;
        case at::kBFloat16: return SRU_BF16;
        case at::kDouble: return SRU_F64;
        default: TORCH_CHECK(false, "sru_cuda: unsupported dtype ", t);
    }
    return -1;
}

const void *ptr(const Tensor &t) { return t.defined() ? t.data_ptr() : nullptr; }

struct Prepared {
    Tensor u, x, wc, bias, init, mask_c, pad;
    at::ScalarType st, sm;
    int64_t D;
};

Prepared prepare(const Tensor &U, const OptTensor &x, const Tensor &weight_c, const Tensor &bias,
                 const Tensor &c_init, const OptTensor &mask_c, const OptTensor &mask_pad,
                 int64_t hidden, int dirs, bool custom, int skip_type) {
    TORCH_CHECK(U.is_cuda(), "sru_cuda: U must be a CUDA tensor (this library has no CPU path)");
    Prepared p;
    p.st = U.scalar_type();
    p.sm = (p.st == at::kDouble) ? at::kDouble : at::kFloat;
    p.D = hidden * dirs;
    p.u = U.contiguous();
    if (skip_type == 1) {
        TORCH_CHECK(x.has_value(), "sru_cuda: skip_type 1 needs x");
        p.x = x.value().to(p.st).contiguous();
    }
    p.wc = weight_c.to(custom ? p.st : p.sm).contiguous();
    p.bias = bias.to(p.sm).contiguous();
    p.init = c_init.to(p.sm).contiguous();
    if (mask_c.has_value()) p.mask_c = mask_c.value().to(p.sm).contiguous();
    if (mask_pad.has_value()) p.pad = mask_pad.value().to(at::kBool).contiguous();
    return p;
}

std::vector<Tensor> forward_impl(const Tensor &U, const OptTensor &x, const Tensor &weight_c,
                                 const Tensor &bias, const Tensor &c_init, const OptTensor &mask_c,
                                 const OptTensor &mask_pad, int64_t length, int64_t batch, int64_t hidden,
                                 int dirs, int64_t k, int64_t act, int64_t skip, int64_t custom) {
    Prepared p = prepare(U, x, weight_c, bias, c_init, mask_c, mask_pad, hidden, dirs, custom != 0, (int)skip);
    c10::cuda::CUDAGuard guard(U.device());
    Tensor h = at::empty({length, batch, p.D}, U.options());
    Tensor c = at::empty({length, batch, p.D}, U.options());
    const int code = dtype_code(p.st);
    const int rc = sru_b200_scan_forward(
        h.data_ptr(), c.data_ptr(), nullptr, ptr(p.u), ptr(p.x), ptr(p.wc), ptr(p.bias), ptr(p.init),
        ptr(p.mask_c), static_cast<const uint8_t *>(ptr(p.pad)), length, batch, hidden, dirs, (int)k,
        (int)act, (int)skip, (int)custom, 1.0, code, code, at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "sru_cuda forward failed: ", sru_b200_last_error());
    return {h, c};
}

std::vector<Tensor> backward_impl(const Tensor &U, const OptTensor &x, const Tensor &weight_c,
                                  const Tensor &bias, const Tensor &c_init, const OptTensor &mask_c,
                                  const OptTensor &mask_pad, const Tensor &c, const Tensor &grad_h,
                                  const Tensor &grad_last, int64_t length, int64_t batch, int64_t hidden,
                                  int dirs, int64_t k, int64_t act, int64_t skip, int64_t custom) {
    Prepared p = prepare(U, x, weight_c, bias, c_init, mask_c, mask_pad, hidden, dirs, custom != 0, (int)skip);
    c10::cuda::CUDAGuard guard(U.device());
    const auto small = U.options().dtype(p.sm);
    Tensor c_hist = c.to(p.st).contiguous();
    Tensor gh = grad_h.to(p.st).contiguous();
    Tensor gl = grad_last.to(p.sm).contiguous();
    Tensor grad_u = at::empty_like(p.u);
    Tensor grad_x = (skip == 1) ? at::empty({length, batch, p.D}, U.options()) : at::zeros({1});
    Tensor grad_wc = custom ? at::empty({length, batch, p.D * 2}, U.options()) : at::empty({2, 1, p.D}, small);
    Tensor grad_bias = at::empty({2, 1, p.D}, small);
    Tensor grad_init = at::empty({batch, p.D}, small);
    const int code = dtype_code(p.st);
    const size_t wbytes = sru_b200_scan_backward_workspace_bytes(length, batch, hidden, dirs, (int)k, code);
    Tensor ws = at::empty({(int64_t)std::max<size_t>(wbytes, 16)}, U.options().dtype(at::kByte));
    const int rc = sru_b200_scan_backward(
        grad_u.data_ptr(), skip == 1 ? grad_x.data_ptr() : nullptr, grad_wc.data_ptr(), grad_bias.data_ptr(),
        grad_init.data_ptr(), ptr(p.u), ptr(p.x), ptr(p.wc), ptr(p.bias), ptr(p.init), ptr(p.mask_c),
        static_cast<const uint8_t *>(ptr(p.pad)), ptr(c_hist), ptr(gh), ptr(gl), length, batch, hidden, dirs,
        (int)k, (int)act, (int)skip, (int)custom, 1.0, code, code, ws.data_ptr(), (size_t)ws.numel(),
        at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "sru_cuda backward failed: ", sru_b200_last_error());
    return {grad_u, grad_x, grad_wc.to(p.st), grad_bias.to(p.st), grad_init.to(p.st)};
}

// ---- the eight operators, argument lists of sru_cuda_impl.cpp:177-518 ----
std::vector<Tensor> sru_forward_simple(const Tensor &U, const OptTensor &x, const Tensor &weight_c,
                                       const Tensor &bias, const Tensor &c_init, const OptTensor &mask_c,
                                       const OptTensor &mask_pad, int64_t length, int64_t batch_size,
                                       int64_t hidden_size) {
    return forward_impl(U, x, weight_c, bias, c_init, mask_c, mask_pad, length, batch_size, hidden_size, 1, 3, 0, 1, 0);
}
std::vector<Tensor> sru_bi_forward_simple(const Tensor &U, const OptTensor &x, const Tensor &weight_c,
                                          const Tensor &bias, const Tensor &c_init, const OptTensor &mask_c,
                                          const OptTensor &mask_pad, int64_t length, int64_t batch_size,
                                          int64_t hidden_size) {
    return forward_impl(U, x, weight_c, bias, c_init, mask_c, mask_pad, length, batch_size, hidden_size, 2, 3, 0, 1, 0);
}
std::vector<Tensor> sru_forward(const Tensor &U, const OptTensor &x, const Tensor &weight_c, const Tensor &bias,
                                const Tensor &c_init, const OptTensor &mask_c, const OptTensor &mask_pad,
                                int64_t length, int64_t batch_size, int64_t hidden_size, int64_t k,
                                int64_t activation_type, int64_t skip_type, int64_t is_custom) {
    return forward_impl(U, x, weight_c, bias, c_init, mask_c, mask_pad, length, batch_size, hidden_size, 1, k,
                        activation_type, skip_type, is_custom);
}
std::vector<Tensor> sru_bi_forward(const Tensor &U, const OptTensor &x, const Tensor &weight_c, const Tensor &bias,
                                   const Tensor &c_init, const OptTensor &mask_c, const OptTensor &mask_pad,
                                   int64_t length, int64_t batch_size, int64_t hidden_size, int64_t k,
                                   int64_t activation_type, int64_t skip_type, int64_t is_custom) {
    return forward_impl(U, x, weight_c, bias, c_init, mask_c, mask_pad, length, batch_size, hidden_size, 2, k,
                        activation_type, skip_type, is_custom);
}
std::vector<Tensor> sru_backward_simple(const Tensor &U, const OptTensor &x, const Tensor &weight_c,
                                        const Tensor &bias, const Tensor &c_init, const OptTensor &mask_c,
                                        const OptTensor &mask_pad, const Tensor &c, const Tensor &grad_h,
                                        const Tensor &grad_last, int64_t length, int64_t batch_size,
                                        int64_t hidden_size) {
    return backward_impl(U, x, weight_c, bias, c_init, mask_c, mask_pad, c, grad_h, grad_last, length, batch_size,
                         hidden_size, 1, 3, 0, 1, 0);
}
std::vector<Tensor> sru_bi_backward_simple(const Tensor &U, const OptTensor &x, const Tensor &weight_c,
                                           const Tensor &bias, const Tensor &c_init, const OptTensor &mask_c,
                                           const OptTensor &mask_pad, const Tensor &c, const Tensor &grad_h,
                                           const Tensor &grad_last, int64_t length, int64_t batch_size,
                                           int64_t hidden_size) {
    return backward_impl(U, x, weight_c, bias, c_init, mask_c, mask_pad, c, grad_h, grad_last, length, batch_size,
                         hidden_size, 2, 3, 0, 1, 0);
}
std::vector<Tensor> sru_backward(const Tensor &U, const OptTensor &x, const Tensor &weight_c, const Tensor &bias,
                                 const Tensor &c_init, const OptTensor &mask_c, const OptTensor &mask_pad,
                                 const Tensor &c, const Tensor &grad_h, const Tensor &grad_last, int64_t length,
                                 int64_t batch_size, int64_t hidden_size, int64_t k, int64_t activation_type,
                                 int64_t skip_type, int64_t is_custom) {
    return backward_impl(U, x, weight_c, bias, c_init, mask_c, mask_pad, c, grad_h, grad_last, length, batch_size,
                         hidden_size, 1, k, activation_type, skip_type, is_custom);
}
std::vector<Tensor> sru_bi_backward(const Tensor &U, const OptTensor &x, const Tensor &weight_c, const Tensor &bias,
                                    const Tensor &c_init, const OptTensor &mask_c, const OptTensor &mask_pad,
                                    const Tensor &c, const Tensor &grad_h, const Tensor &grad_last, int64_t length,
                                    int64_t batch_size, int64_t hidden_size, int64_t k, int64_t activation_type,
                                    int64_t skip_type, int64_t is_custom) {
    return backward_impl(U, x, weight_c, bias, c_init, mask_c, mask_pad, c, grad_h, grad_last, length, batch_size,
                         hidden_size, 2, k, activation_type, skip_type, is_custom);
}

// ---- operators of this package's own namespace: what the scripted module calls instead of library kernels ----

// y = x (M, K) @ w (K, N) [+ col_bias] on the tcgen05 GEMM for 16-bit CUDA operands whose shapes the tensor-map
// loads take (K, N multiples of 8, 16-byte aligned rows); anything else is the library product, like Tensor.mm.
Tensor b200_gemm(const Tensor &x, const Tensor &w, const OptTensor &col_bias) {
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(0), "sru_b200::gemm: shapes (M,K) x (K,N) expected");
    const auto st = x.scalar_type();
    const bool sixteen = (st == at::kHalf || st == at::kBFloat16) && w.scalar_type() == st;
    const int64_t m = x.size(0), k = x.size(1), n = w.size(1);
    if (!(x.is_cuda() && sixteen && k % 8 == 0 && n % 8 == 0 && m > 0 && k > 0)) {
        Tensor out = at::mm(x, w);
        if (col_bias.has_value()) out = out + col_bias.value().to(out.scalar_type());
        return out;
    }
    c10::cuda::CUDAGuard guard(x.device());
    Tensor xc = x.contiguous(), wc = w.contiguous();
    Tensor bias;
    if (col_bias.has_value()) bias = col_bias.value().to(at::kFloat).contiguous();
    Tensor out = at::empty({m, n}, x.options());
    const int code = dtype_code(st);
    const size_t wbytes = sru_b200_gemm_workspace_bytes(m, n, k, bias.defined() ? 1 : 0);
    Tensor ws = at::empty({(int64_t)std::max<size_t>(wbytes, 16)}, x.options().dtype(at::kByte));
    const int rc = sru_b200_gemm_ws(out.data_ptr(), xc.data_ptr(), wc.data_ptr(),
                                    bias.defined() ? bias.data_ptr<float>() : nullptr, m, n, k, k, n, n, 0, 0, code,
                                    code, 0, ws.data_ptr(), wbytes, at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "sru_b200::gemm failed: ", sru_b200_last_error());
    return out;
}

// The layer's gate bias (2 * width) as the col_bias vector of U's gate-innermost columns.
Tensor b200_gate_bias_columns(const Tensor &bias, int64_t width, int64_t k) {
    TORCH_CHECK(bias.is_cuda() && bias.numel() == 2 * width, "sru_b200::gate_bias_columns: CUDA bias of 2*width expected");
    c10::cuda::CUDAGuard guard(bias.device());
    Tensor b = bias.to(at::kFloat).contiguous();
    Tensor out = at::empty({width * k}, b.options());
    const int rc = sru_b200_gate_bias_columns(out.data_ptr<float>(), b.data_ptr<float>(), width, (int)k,
                                              at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "sru_b200::gate_bias_columns failed: ", sru_b200_last_error());
    return out;
}

// Layer normalisation over the last dimension, forward only (the scripted module is an inference path); row lengths
// the kernels do not take go to the library operator.
Tensor b200_layer_norm(const Tensor &x, const OptTensor &weight, const OptTensor &bias, double eps) {
    const int64_t n = x.size(-1);
    const auto st = x.scalar_type();
    const bool f32 = st == at::kFloat, sixteen = (st == at::kHalf || st == at::kBFloat16);
    if (!(x.is_cuda() && (f32 || sixteen) && n > 0 && n <= 4096 && n % (f32 ? 4 : 8) == 0 && x.numel() > 0)) {
        return at::layer_norm(x, {n}, weight, bias, eps);
    }
    c10::cuda::CUDAGuard guard(x.device());
    Tensor xc = x.contiguous();
    Tensor w, b;
    if (weight.has_value()) w = weight.value().to(at::kFloat).contiguous();
    if (bias.has_value()) b = bias.value().to(at::kFloat).contiguous();
    Tensor y = at::empty_like(xc);
    const int code = dtype_code(st);
    const int rc = sru_b200_layer_norm_forward(y.data_ptr(), nullptr, nullptr, xc.data_ptr(),
                                               w.defined() ? w.data_ptr<float>() : nullptr,
                                               b.defined() ? b.data_ptr<float>() : nullptr, xc.numel() / n, n, eps, code,
                                               code, at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "sru_b200::layer_norm failed: ", sru_b200_last_error());
    return y;
}

// The layer loop of an inference forward as ONE call (sru/modules.py:617-646 is a Python loop over the layers, each
// of them a matrix product and a recurrence launch, with a layer norm before or after when the stack has one): per
// layer the optional pre-norm (written in the compute type), the gate bias laid out for the product's epilogue,
// U = x W (+ bias) on the tcgen05 GEMM, the scan (U, and x as the highway input when k = 3; h in the compute type, the
// layer's final state in float32) and the optional post-norm.  For stacks of plain layers (no factorised projection,
// no custom module, identity activation) whose shapes the kernels take (rows, input width and D*k multiples of 8,
// normalised rows of at most 4096 elements); the Python module checks that and otherwise keeps its own loop.
// x is float32 (autocast: the first layer norm then reads the unrounded rows, as the module's does) or already
// in the compute type.  weights[i] may already be in the compute type and col_bias[i] may hold the gate bias laid out
// over U's columns (a caller that serves many requests keeps both between calls; with no elements it is laid out
// here).  ln_weight[i] / ln_bias[i] with no elements mean "no affine part"; has_norm[i] says whether
// layer i has a norm at all.  Same kernels with the same arguments as the Python loop: identical results.
Tensor stack_layer_norm(const Tensor &t, const Tensor &w, const Tensor &b, double eps, at::ScalarType out, void *stream) {
    const int64_t n = t.size(-1);
    Tensor tc = t.contiguous();
    Tensor y = at::empty(tc.sizes(), tc.options().dtype(out));
    Tensor wf, bf;
    if (w.numel() > 0) wf = w.to(at::kFloat).contiguous();
    if (b.numel() > 0) bf = b.to(at::kFloat).contiguous();
    const int rc = sru_b200_layer_norm_forward(y.data_ptr(), nullptr, nullptr, tc.data_ptr(),
                                               wf.defined() ? wf.data_ptr<float>() : nullptr,
                                               bf.defined() ? bf.data_ptr<float>() : nullptr, tc.numel() / n, n, eps,
                                               dtype_code(tc.scalar_type()), dtype_code(out), stream);
    TORCH_CHECK(rc == 0, "sru_b200::stack_forward: ", sru_b200_last_error());
    return y;
}

std::vector<Tensor> b200_stack_forward(const Tensor &x, std::vector<Tensor> weights, std::vector<Tensor> weight_c,
                                       std::vector<Tensor> bias, std::vector<double> scale_x, const OptTensor &c0,
                                       const OptTensor &mask_pad, int64_t hidden, bool bidirectional,
                                       std::vector<int64_t> ks, std::vector<int64_t> skips, bool half_is_fp16,
                                       std::vector<int64_t> has_norm, std::vector<Tensor> ln_weight,
                                       std::vector<Tensor> ln_bias, std::vector<double> ln_eps, bool normalize_after,
                                       std::vector<Tensor> col_biases) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 3, "sru_b200::stack_forward: x must be a CUDA tensor (length, batch, width)");
    const at::ScalarType st = half_is_fp16 ? at::kHalf : at::kBFloat16;
    TORCH_CHECK(x.scalar_type() == st || x.scalar_type() == at::kFloat,
                "sru_b200::stack_forward: x must be float32 or of the compute type");
    const size_t n = weights.size();
    TORCH_CHECK(n > 0 && weight_c.size() == n && bias.size() == n && scale_x.size() == n && ks.size() == n &&
                skips.size() == n && has_norm.size() == n && ln_weight.size() == n && ln_bias.size() == n &&
                ln_eps.size() == n && col_biases.size() == n,
                "sru_b200::stack_forward: one entry per layer expected in every list");
    c10::cuda::CUDAGuard guard(x.device());
    void *stream = at::cuda::getCurrentCUDAStream().stream();
    const int dirs = bidirectional ? 2 : 1;
    const int64_t L = x.size(0), B = x.size(1), D = hidden * dirs, M = L * B;
    TORCH_CHECK(M > 0 && M % 8 == 0, "sru_b200::stack_forward: length * batch must be a positive multiple of 8");
    const int code = dtype_code(st);
    const auto f32 = x.options().dtype(at::kFloat);
    const auto o16 = x.options().dtype(st);
    Tensor pad;
    if (mask_pad.has_value()) {
        pad = mask_pad.value().to(at::kBool).contiguous();
        TORCH_CHECK(pad.dim() == 2 && pad.size(0) == L && pad.size(1) == B, "sru_b200::stack_forward: mask_pad must be (length, batch)");
    }
    Tensor init;
    if (c0.has_value()) {
        init = c0.value().to(at::kFloat).contiguous();
        TORCH_CHECK(init.dim() == 3 && init.size(0) == (int64_t)n && init.size(1) == B && init.size(2) == D,
                    "sru_b200::stack_forward: c0 must be (layers, batch, width)");
    }
    Tensor c_stack = at::empty({(int64_t)n, B, D}, f32);
    Tensor cur = x.contiguous();       // float32 only before the first layer
    for (size_t i = 0; i < n; ++i) {
        const int64_t in = cur.size(2), k = ks[i], N = D * k, skip = skips[i];
        TORCH_CHECK(weights[i].dim() == 2 && weights[i].size(0) == in && weights[i].size(1) == N,
                    "sru_b200::stack_forward: weight of layer ", i, " must be (", in, ", ", N, ")");
        TORCH_CHECK(in % 8 == 0 && N % 8 == 0, "sru_b200::stack_forward: widths must be multiples of 8");
        TORCH_CHECK((k == 3 || k == 4) && (skip == 0 || (skip == 1 && k == 3 && in == D) || (skip == 2 && k == 4)),
                    "sru_b200::stack_forward: layer ", i, " has k = ", k, " with skip type ", skip);
        Tensor w = weights[i].to(st).contiguous();
        Tensor wc = weight_c[i].to(at::kFloat).contiguous();
        Tensor b = bias[i].to(at::kFloat).contiguous();
        TORCH_CHECK(wc.numel() == 2 * D && b.numel() == 2 * D, "sru_b200::stack_forward: weight_c and bias hold 2 * width values");
        // operand of the product: the normalised rows, or the input in the compute type
        Tensor a_in;
        if (has_norm[i] && !normalize_after) a_in = stack_layer_norm(cur, ln_weight[i], ln_bias[i], ln_eps[i], st, stream);
        else a_in = (cur.scalar_type() == st) ? cur : cur.to(st);
        // the gate bias over U's columns: handed in by a caller that keeps it between calls, else laid out here
        Tensor col_bias = col_biases[i];
        int rc = 0;
        if (col_bias.numel() == 0) {
            col_bias = at::empty({N}, f32);
            rc = sru_b200_gate_bias_columns(col_bias.data_ptr<float>(), b.data_ptr<float>(), D, (int)k, stream);
            TORCH_CHECK(rc == 0, "sru_b200::stack_forward: ", sru_b200_last_error());
        } else {
            TORCH_CHECK(col_bias.is_cuda() && col_bias.scalar_type() == at::kFloat && col_bias.numel() == N &&
                        col_bias.is_contiguous(), "sru_b200::stack_forward: col_bias of layer ", i, " must be float[", N, "]");
        }
        Tensor u = at::empty({M, N}, o16);
        const size_t wbytes = sru_b200_gemm_workspace_bytes(M, N, in, 1);
        Tensor ws = at::empty({(int64_t)std::max<size_t>(wbytes, 16)}, x.options().dtype(at::kByte));
        rc = sru_b200_gemm_ws(u.data_ptr(), a_in.data_ptr(), w.data_ptr(), col_bias.data_ptr<float>(), M, N, in, in, N, N,
                              0, 0, code, code, 0, ws.data_ptr(), wbytes, stream);
        TORCH_CHECK(rc == 0, "sru_b200::stack_forward: ", sru_b200_last_error());
        Tensor hx;                      // the highway input: the layer's (un-normalised) input in the compute type
        if (skip == 1) hx = (cur.scalar_type() == st) ? cur : cur.to(st);
        Tensor h = at::empty({L, B, D}, o16);
        rc = sru_b200_scan_forward(h.data_ptr(), nullptr, c_stack[i].data_ptr(), u.data_ptr(), ptr(hx), wc.data_ptr(),
                                   nullptr, init.defined() ? init[i].data_ptr() : nullptr, nullptr,
                                   static_cast<const uint8_t *>(ptr(pad)), L, B, hidden, dirs, (int)k, 0, (int)skip, 0,
                                   scale_x[i], code, SRU_F32, stream);
        TORCH_CHECK(rc == 0, "sru_b200::stack_forward: ", sru_b200_last_error());
        if (has_norm[i] && normalize_after) h = stack_layer_norm(h, ln_weight[i], ln_bias[i], ln_eps[i], st, stream);
        cur = h;
    }
    return {cur, c_stack};
}

}  // namespace

TORCH_LIBRARY(sru_b200, m) {
    m.def("stack_forward(Tensor x, Tensor[] weights, Tensor[] weight_c, Tensor[] bias, float[] scale_x, Tensor? c0, "
          "Tensor? mask_pad, int hidden_size, bool bidirectional, int[] k, int[] skip_type, bool half_is_fp16, "
          "int[] has_norm, Tensor[] ln_weight, Tensor[] ln_bias, float[] ln_eps, bool normalize_after, Tensor[] col_bias) "
          "-> Tensor[]",
          &b200_stack_forward);
    m.def("gemm(Tensor x, Tensor w, Tensor? col_bias) -> Tensor", &b200_gemm);
    m.def("gate_bias_columns(Tensor bias, int width, int k) -> Tensor", &b200_gate_bias_columns);
    m.def("layer_norm(Tensor x, Tensor? weight, Tensor? bias, float eps) -> Tensor", &b200_layer_norm);
}

TORCH_LIBRARY(sru_cuda, m) {
    m.def("sru_forward_simple", &sru_forward_simple);
    m.def("sru_backward_simple", &sru_backward_simple);
    m.def("sru_bi_forward_simple", &sru_bi_forward_simple);
    m.def("sru_bi_backward_simple", &sru_bi_backward_simple);
    m.def("sru_forward", &sru_forward);
    m.def("sru_backward", &sru_backward);
    m.def("sru_bi_forward", &sru_bi_forward);
    m.def("sru_bi_backward", &sru_bi_backward);
}
