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

}  // namespace

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
