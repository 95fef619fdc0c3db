"""Operator layer of the SRU hot path on B200: the light-recurrence scan through the C ABI.

Mirrors the reference's operator interface for this path:

* ``elementwise_recurrence_gpu``  -- sru/ops.py:97-142 (same arguments, same return value)
* ``ElementwiseRecurrence``       -- sru/cuda_functional.py:156-261 (autograd glue)
* ``elementwise_recurrence_forward`` -- sru/cuda_functional.py:37-153 (returns h, last_hidden, c)

Differences, all inside the boundary: the kernels read U / x / grad_h in their storage
dtype and compute in fp32 registers (no fp32 copies of U); ``x * scale_x``, the
bidirectional ``last_hidden`` gather, ``grad_x *= scale_x`` and the batch reduction of
``grad_weight_c`` / ``grad_bias`` happen inside the kernels; outputs are not memset.
There is no CPU path here: tensors must be CUDA tensors and the native library must load.
"""
from typing import List, Optional, Tuple

import torch
from torch import Tensor
from torch.autograd import Function

from . import _lib

# How a 16-bit U (from an autocast GEMM) is handled.
#   "native":    scan reads/writes the 16-bit storage dtype directly, h comes back in that dtype.
#   "reference": U and x are first cast to fp32 exactly as sru/ops.py:116-127 does (fp16 when
#                amp_recurrence_fp16 and U is fp16), h comes back in that cast dtype.
_amp_mode = "native"
# Storage of the saved state history c (L,B,D) when U is 16-bit: "float32" or "storage".
_c_hist_dtype = "float32"


def set_amp_mode(mode: str) -> None:
    global _amp_mode
    if mode not in ("native", "reference"):
        raise ValueError("amp mode must be 'native' or 'reference'")
    _amp_mode = mode


def get_amp_mode() -> str:
    return _amp_mode


def set_c_hist_dtype(kind: str) -> None:
    global _c_hist_dtype
    if kind not in ("float32", "storage"):
        raise ValueError("c_hist dtype must be 'float32' or 'storage'")
    _c_hist_dtype = kind


# Callables invoked (no arguments) right after a backward scan has been enqueued on the current stream.  The
# gradient all-reducer of distributed.py uses this to start a finished layer's collective behind the next
# layer's scan instead of beside it.
_scan_backward_listeners: list = []


def add_scan_backward_listener(fn) -> None:
    if fn not in _scan_backward_listeners:
        _scan_backward_listeners.append(fn)


def remove_scan_backward_listener(fn) -> None:
    if fn in _scan_backward_listeners:
        _scan_backward_listeners.remove(fn)


def _small_dtype(storage: torch.dtype) -> torch.dtype:
    return torch.float64 if storage == torch.float64 else torch.float32


def _c_dtype_for(storage: torch.dtype) -> torch.dtype:
    if storage in (torch.float16, torch.bfloat16) and _c_hist_dtype == "float32":
        return torch.float32
    return storage


def _require_cuda(t: Tensor, name: str) -> None:
    if not t.is_cuda:
        raise _lib.SruB200Error("%s must be a CUDA tensor: sru_b200 has no CPU path" % name)


def _geometry(u: Tensor, x: Tensor, d: int, bidirectional: bool, has_skip_term: bool, weight_c: Tensor):
    dirs = 2 if bidirectional else 1
    length = x.size(0) if x.dim() == 3 else 1
    batch = x.size(-2)
    k = u.size(-1) // d // dirs
    skip_type = 0 if not has_skip_term else (1 if k == 3 else 2)
    is_custom = 1 if weight_c.dim() > 1 else 0
    return length, batch, dirs, k, skip_type, is_custom


def scan_forward(u: Tensor, x: Optional[Tensor], weight_c: Tensor, bias: Optional[Tensor],
                 c_init: Optional[Tensor], mask_c: Optional[Tensor], mask_pad: Optional[Tensor],
                 length: int, batch: int, d: int, dirs: int, k: int, activation_type: int,
                 skip_type: int, is_custom: int, scale_x: float, need_c_hist: bool = True,
                 c_dtype: Optional[torch.dtype] = None) -> Tuple[Tensor, Optional[Tensor], Tensor]:
    """Raw forward call.  u is (L,B,D*k) in the storage dtype; returns h, c_hist (or None), c_last."""
    _require_cuda(u, "U")
    st = u.dtype
    sm = _small_dtype(st)
    D = d * dirs
    if c_dtype is None:
        c_dtype = _c_dtype_for(st)
    h = torch.empty(length, batch, D, dtype=st, device=u.device)
    c_hist = torch.empty(length, batch, D, dtype=c_dtype, device=u.device) if need_c_hist else None
    c_last = torch.empty(batch, D, dtype=sm, device=u.device)
    if length == 0 or batch == 0:
        if c_init is not None:
            c_last.copy_(c_init.reshape(batch, D))
        else:
            c_last.zero_()
        return h, c_hist, c_last
    with torch.cuda.device(u.device):
        _lib.call(
            "scan_fwd" if need_c_hist else "scan_fwd_infer", 1, _lib.lib().sru_b200_scan_forward,
            _lib.ptr(h), _lib.ptr(c_hist), _lib.ptr(c_last), _lib.ptr(u), _lib.ptr(x),
            _lib.ptr(weight_c), _lib.ptr(bias), _lib.ptr(c_init), _lib.ptr(mask_c), _lib.ptr(mask_pad),
            length, batch, d, dirs, k, activation_type, skip_type, is_custom, float(scale_x),
            _lib.DTYPE_CODE[st], _lib.DTYPE_CODE[c_dtype], _lib.current_stream_ptr(u.device))
    return h, c_hist, c_last


def scan_backward(u, x, weight_c, bias, c_init, mask_c, mask_pad, c_hist, grad_h, grad_last,
                  length, batch, d, dirs, k, activation_type, skip_type, is_custom, scale_x):
    """Raw backward call.  Returns grad_u, grad_x (or None), grad_wc, grad_bias (2*D), grad_init."""
    st = u.dtype
    sm = _small_dtype(st)
    D = d * dirs
    dev = u.device
    grad_u = torch.empty_like(u)
    grad_x = torch.empty(length, batch, D, dtype=st, device=dev) if skip_type == 1 else None
    if is_custom:
        grad_wc = torch.empty(length, batch, D * 2, dtype=st, device=dev)
    else:
        grad_wc = torch.empty(2 * D, dtype=sm, device=dev)
    grad_bias = torch.empty(2 * D, dtype=sm, device=dev)
    grad_init = torch.empty(batch, D, dtype=sm, device=dev)
    if length == 0 or batch == 0:
        grad_wc.zero_(); grad_bias.zero_()
        if grad_last is not None:
            grad_init.copy_(grad_last)
        else:
            grad_init.zero_()
        return grad_u, grad_x, grad_wc, grad_bias, grad_init
    L = _lib.lib()
    code = _lib.DTYPE_CODE[st]
    nbytes = L.sru_b200_scan_backward_workspace_bytes(length, batch, d, dirs, k, code)
    workspace = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.call(
            "scan_bwd", 2, L.sru_b200_scan_backward,
            _lib.ptr(grad_u), _lib.ptr(grad_x), _lib.ptr(grad_wc), _lib.ptr(grad_bias), _lib.ptr(grad_init),
            _lib.ptr(u), _lib.ptr(x), _lib.ptr(weight_c), _lib.ptr(bias), _lib.ptr(c_init),
            _lib.ptr(mask_c), _lib.ptr(mask_pad), _lib.ptr(c_hist), _lib.ptr(grad_h), _lib.ptr(grad_last),
            length, batch, d, dirs, k, activation_type, skip_type, is_custom, float(scale_x),
            code, _lib.DTYPE_CODE[c_hist.dtype], _lib.ptr(workspace), workspace.numel(),
            _lib.current_stream_ptr(dev))
    return grad_u, grad_x, grad_wc, grad_bias, grad_init


def _prep_small(t: Optional[Tensor], dtype: torch.dtype) -> Optional[Tensor]:
    if t is None:
        return None
    return t.detach().to(dtype).contiguous()


def _scale_value(scale_x: Optional[Tensor]) -> float:
    """The scalar the kernels take for ``scale_x`` (sru/cuda_functional.py:73-78).  Reading a device tensor
    synchronises the stream, so the value is remembered on the tensor object, keyed by the tensor's storage
    address and version counter, and read again after any in-place change autograd can see (``copy_``,
    ``fill_``, indexing assignment, ``load_state_dict``).  A write through ``.data`` does not move the version
    counter: ``SRUCell`` drops the remembered value in ``reset_parameters`` and when a state dict is loaded,
    and code that pokes ``scale_x.data`` itself calls ``forget_scale(scale_x)`` afterwards."""
    if scale_x is None:
        return 1.0
    key = (scale_x.data_ptr(), scale_x._version)
    cached = getattr(scale_x, "_sru_b200_scalar", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    value = float(scale_x.reshape(-1)[0])
    try:
        scale_x._sru_b200_scalar = (key, value)
    except Exception:       # tensors that refuse attributes are simply read every time
        pass
    return value


def _convert(t: Tensor, dtype: torch.dtype) -> Tensor:
    """t in ``dtype`` through ``sru_b200_convert`` (float32 <-> fp16 / bf16, contiguous CUDA tensors)."""
    out = torch.empty(t.shape, dtype=dtype, device=t.device)
    if t.numel():
        with torch.cuda.device(t.device):
            _lib.call("convert", 1 if t.numel() % 8 == 0 else 2, _lib.lib().sru_b200_convert, _lib.ptr(out), _lib.ptr(t),
                      t.numel(), _lib.DTYPE_CODE[t.dtype], _lib.DTYPE_CODE[dtype], _lib.current_stream_ptr(t.device))
    return out


class _Widen(torch.autograd.Function):
    """16-bit -> float32 with the adjoint float32 -> 16-bit, both on this package's conversion kernel."""

    @staticmethod
    def forward(ctx, t):
        ctx.src_dtype = t.dtype
        return _convert(t, torch.float32)

    @staticmethod
    def backward(ctx, grad):
        g = grad if grad.is_contiguous() else grad.contiguous()
        if g.dtype != torch.float32:
            return g.to(ctx.src_dtype)
        return _convert(g, ctx.src_dtype)


def widen_to_float32(t: Tensor) -> Tensor:
    """``t.float()`` for the 16-bit h the module hands back as float32 (the reference's return type under 16-bit
    autocast, sru/ops.py:116-127).  The framework's converting copy of a large tensor runs at about a quarter of the HBM
    bandwidth; this one is bound by it.  Anything the kernel does not take (CPU, non-contiguous, unaligned, other
    types) is converted by the framework."""
    if (t.is_cuda and t.dtype in (torch.float16, torch.bfloat16) and t.is_contiguous() and t.data_ptr() % 16 == 0
            and not torch.jit.is_scripting()):
        with torch.autocast("cuda", enabled=False):
            return _Widen.apply(t)
    return t.float()


def forget_scale(scale_x: Optional[Tensor]) -> None:
    """Drops the remembered scalar of ``scale_x`` (call after writing to it through ``.data``)."""
    if scale_x is not None and hasattr(scale_x, "_sru_b200_scalar"):
        try:
            del scale_x._sru_b200_scalar
        except Exception:
            pass


class ElementwiseRecurrence(Function):
    """Autograd function of the scan; argument order of sru/cuda_functional.py:158-169."""

    @staticmethod
    def forward(ctx, u, x, weight_c, bias, init, activation_type, d_out, bidirectional,
                has_skip_term, scale_x, mask_c=None, mask_pad=None, grad_link=None, bias_in_u=False):
        length, batch, dirs, k, skip_type, is_custom = _geometry(u, x, d_out, bidirectional,
                                                                 has_skip_term, weight_c)
        ctx.set_materialize_grads(False)    # no zero tensor is built for the (usually unused) gradient of the final state
        st = u.dtype
        sm = _small_dtype(st)
        D = d_out * dirs
        u_c = u.detach().contiguous()
        x_c = x.detach().to(st).contiguous() if skip_type == 1 else None
        wc_c = weight_c.detach().to(st if is_custom else sm).contiguous()
        # bias_in_u: the producer of U has already added the bias (GEMM epilogue); the kernels then take no bias,
        # and the backward still delivers grad_bias (the sums it forms do not depend on where the bias was added)
        bias_c = None if bias_in_u else _prep_small(bias, sm)
        init_c = _prep_small(init, sm)
        mask_c_c = _prep_small(mask_c, sm)
        pad_c = mask_pad.bool().contiguous() if mask_pad is not None else None
        scale = _scale_value(scale_x)
        need_hist = any(ctx.needs_input_grad[:5])
        h, c_hist, c_last = scan_forward(u_c.view(length, batch, D * k), x_c, wc_c, bias_c, init_c,
                                         mask_c_c, pad_c, length, batch, d_out, dirs, k,
                                         activation_type, skip_type, is_custom, scale, need_hist)
        ctx.meta = (length, batch, d_out, dirs, k, activation_type, skip_type, is_custom, scale)
        ctx.shapes = (u.shape, x.shape, x.dtype, weight_c.shape, weight_c.dtype, bias.dtype,
                      init.shape, init.dtype)
        ctx.save_for_backward(u_c, x_c, wc_c, bias_c, init_c, mask_c_c, pad_c, c_hist)
        # an armed link takes grad_x to the projection's backward (see projection.GradLink); only when the
        # scan reads x as it is, so that its grad_x is the gradient of that very tensor
        ctx.link = grad_link if (grad_link is not None and grad_link.armed and skip_type == 1
                                 and x.dtype == st and x.is_contiguous()) else None
        if x.dim() == 2:
            h = h.squeeze(0)
        return h, c_last

    @staticmethod
    def backward(ctx, grad_h, grad_last):
        u, x, wc, bias, init, mask_c, pad, c_hist = ctx.saved_tensors
        length, batch, d, dirs, k, act, skip_type, is_custom, scale = ctx.meta
        u_shape, x_shape, x_dtype, wc_shape, wc_dtype, bias_dtype, init_shape, init_dtype = ctx.shapes
        D = d * dirs
        st = u.dtype
        sm = _small_dtype(st)
        # gradients autograd did not produce arrive as None (set_materialize_grads(False) in forward): the kernel takes
        # a null grad_last as zeros, and a missing grad_h (only the final state was used) becomes zeros here
        if grad_h is None:
            gh = torch.zeros(length, batch, D, dtype=st, device=u.device)
        else:
            gh = grad_h.to(st).contiguous().view(length, batch, D)
        gl = _prep_small(grad_last, sm)
        grad_u, grad_x, grad_wc, grad_bias, grad_init = scan_backward(
            u.view(length, batch, D * k), x, wc, bias, init, mask_c, pad, c_hist, gh, gl,
            length, batch, d, dirs, k, act, skip_type, is_custom, scale)
        for fn in tuple(_scan_backward_listeners):
            fn()
        grad_u = grad_u.view(u_shape)
        if grad_x is not None:
            if ctx.link is not None:
                ctx.link.grad_x, grad_x = grad_x, None    # the projection's backward adds its dgrad onto it
            else:
                grad_x = grad_x.view(x_shape).to(x_dtype)
        grad_wc = grad_wc.view(wc_shape).to(wc_dtype)
        return (grad_u, grad_x, grad_wc, grad_bias.to(bias_dtype), grad_init.view(init_shape).to(init_dtype),
                None, None, None, None, None, None, None, None, None)


def elementwise_recurrence_forward(u: Tensor, x: Tensor, weight_c: Tensor, bias: Tensor, init: Tensor,
                                   activation_type: int, d_out: int, bidirectional: bool,
                                   has_skip_term: bool, scale_x: Optional[Tensor] = None,
                                   mask_c: Optional[Tensor] = None,
                                   mask_pad: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Tensor]:
    """No-grad forward returning (h, last_hidden, c) as sru/cuda_functional.py:37-153 does."""
    length, batch, dirs, k, skip_type, is_custom = _geometry(u, x, d_out, bidirectional,
                                                             has_skip_term, weight_c)
    st = u.dtype
    sm = _small_dtype(st)
    D = d_out * dirs
    scale = _scale_value(scale_x)
    h, c_hist, c_last = scan_forward(
        u.detach().contiguous().view(length, batch, D * k),
        x.detach().to(st).contiguous() if skip_type == 1 else None,
        weight_c.detach().to(st if is_custom else sm).contiguous(), _prep_small(bias, sm),
        _prep_small(init, sm), _prep_small(mask_c, sm),
        mask_pad.bool().contiguous() if mask_pad is not None else None,
        length, batch, d_out, dirs, k, activation_type, skip_type, is_custom, scale, True)
    if x.dim() == 2:
        h, c_hist = h.squeeze(0), c_hist.squeeze(0)
    return h, c_last, c_hist


def elementwise_recurrence_gpu(U: Tensor, x: Tensor, weight_c: Tensor, bias: Tensor, c_init: Tensor,
                               activation_type: int, hidden_size: int, bidirectional: bool,
                               has_skip_term: bool, scale_x: Optional[Tensor] = None,
                               dropout_mask_c: Optional[Tensor] = None,
                               mask_pad: Optional[Tensor] = None,
                               amp_recurrence_fp16: bool = False,
                               grad_link=None, bias_in_u: bool = False) -> List[Tensor]:
    """Elementwise recurrence of SRU on the GPU; signature of sru/ops.py:98-110, plus ``grad_link``
    (a projection.GradLink armed by the projection that produced U from the same x; optional) and
    ``bias_in_u`` (U already contains the gate bias; ``bias`` is then only the tensor grad_bias belongs to).

    Returns ``[h, last_c]``.  In "reference" amp mode the casts of sru/ops.py:116-127 are
    applied first, so dtypes of the results equal the reference's; in "native" mode (default)
    a 16-bit U is consumed as it is and h has U's dtype; last_c is float32 (see below).
    """
    _require_cuda(U, "U")
    if _amp_mode == "reference":
        if amp_recurrence_fp16 and U.dtype == torch.float16:
            cast = torch.Tensor.half
        else:
            cast = torch.Tensor.float
        U, x, c_init = cast(U), cast(x), cast(c_init)
        grad_link = None      # x is a cast copy here: its gradient is not the GEMM operand's
    # The final state comes back as the reference's does (sru/ops.py:116-124 casts c_init before the scan): half
    # precision with amp_recurrence_fp16 on a half U, float32 otherwise, whatever type c_init had.  A float32
    # state also makes a sequence processed in chunks (state handed from chunk to chunk) bit-identical to one pass.
    c_dtype = torch.float16 if (amp_recurrence_fp16 and U.dtype == torch.float16) else _small_dtype(U.dtype)
    if not torch.is_grad_enabled() or not any(
            t is not None and t.requires_grad for t in (U, x, weight_c, bias, c_init)):
        h, c_last, _ = _forward_nograd(U, x, weight_c, None if bias_in_u else bias, c_init, activation_type,
                                       hidden_size, bidirectional, has_skip_term, scale_x, dropout_mask_c, mask_pad)
        return [h, c_last.to(c_dtype)]
    h, c_last = ElementwiseRecurrence.apply(U, x, weight_c, bias, c_init, activation_type, hidden_size,
                                            bidirectional, has_skip_term, scale_x, dropout_mask_c,
                                            mask_pad, grad_link, bias_in_u)
    return [h, c_last if c_last.dtype == c_dtype else c_last.to(c_dtype)]


def _forward_nograd(U, x, weight_c, bias, c_init, activation_type, hidden_size, bidirectional,
                    has_skip_term, scale_x, mask_c, mask_pad):
    """Inference: no state history is written (5 instead of 6 elements of traffic per column-step)."""
    length, batch, dirs, k, skip_type, is_custom = _geometry(U, x, hidden_size, bidirectional,
                                                             has_skip_term, weight_c)
    st = U.dtype
    sm = _small_dtype(st)
    D = hidden_size * dirs
    scale = _scale_value(scale_x)
    h, _, c_last = scan_forward(
        U.detach().contiguous().view(length, batch, D * k),
        x.detach().to(st).contiguous() if skip_type == 1 else None,
        weight_c.detach().to(st if is_custom else sm).contiguous(), _prep_small(bias, sm),
        _prep_small(c_init, sm), _prep_small(mask_c, sm),
        mask_pad.bool().contiguous() if mask_pad is not None else None,
        length, batch, hidden_size, dirs, k, activation_type, skip_type, is_custom, scale, False)
    if x.dim() == 2:
        h = h.squeeze(0)
    return h, c_last, None
