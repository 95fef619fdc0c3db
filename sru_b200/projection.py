"""The dense projection U = x W of the SRU layer (sru/modules.py:363-378) and its gradients.

16-bit operands (bf16 / fp16, e.g. under autocast) run on this package's tcgen05 GEMM
(``sru_b200_gemm`` of the C ABI): forward ``U = x W``, backward ``grad_x = grad_U W^T`` and
``grad_W = x^T grad_U``, all with fp32 accumulation in tensor memory.  float32 operands CAN run on the
same GEMM through a three-way bfloat16 split (``sru_b200_gemm_f32``, ``set_fp32_on_tensor_cores``);
by default they, float64 and odd shapes are a plain library GEMM (``torch.mm``), because the
split product's accuracy (2e-6 ... 2e-5) does not meet the 1e-5 float32 parity bar for long reductions.
"""
import os
from typing import Optional

import torch
from torch import Tensor
from torch.autograd import Function

from . import _lib

_SIXTEEN = (torch.float16, torch.bfloat16)


_backend = os.environ.get("SRU_B200_GEMM", "tcgen05")     # read once, at import


def gemm_backend() -> str:
    """'tcgen05' (default) or 'library' (torch.mm everywhere; for A/B measurements)."""
    return _backend


def set_gemm_backend(name: str) -> None:
    global _backend
    if name not in ("tcgen05", "library"):
        raise ValueError("gemm backend must be 'tcgen05' or 'library'")
    _backend = name


def gemm(a: Tensor, b: Tensor, trans_a: bool = False, trans_b: bool = False,
         out_dtype: Optional[torch.dtype] = None, col_bias: Optional[Tensor] = None,
         out: Optional[Tensor] = None, accumulate: bool = False, name: Optional[str] = None) -> Tensor:
    """C = op(a) @ op(b) (+ col_bias) on the tcgen05 kernel.  a, b: 2-D, 16-bit, same dtype,
    unit stride in the last dimension.  op(a) is M x K, op(b) is K x N."""
    if a.dtype not in _SIXTEEN or b.dtype != a.dtype:
        raise _lib.SruB200Error("gemm operands must both be bf16 or both fp16")
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    m = a.size(1) if trans_a else a.size(0)
    kd = a.size(0) if trans_a else a.size(1)
    kb = b.size(1) if trans_b else b.size(0)
    n = b.size(0) if trans_b else b.size(1)
    if kd != kb:
        raise _lib.SruB200Error("gemm inner dimensions differ: %d vs %d" % (kd, kb))
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype or a.dtype, device=a.device)
    if m == 0 or n == 0:
        return out
    if kd == 0:
        return out if accumulate else out.zero_()
    bias = None if col_bias is None else col_bias.detach().float().contiguous()
    L = _lib.lib()
    with torch.cuda.device(a.device):
        if name is None:
            name = "gemm_wgrad" if trans_a else ("gemm_dgrad" if trans_b else "gemm_fwd")
        # long reductions into few output tiles are cut into K slabs; the library says how much scratch it wants
        ws_bytes = int(L.sru_b200_gemm_workspace_bytes(m, n, kd, 0 if bias is None else 1))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device) if ws_bytes else None
        _lib.call(
            name, 2 if ws_bytes > 32768 else 1, L.sru_b200_gemm_ws,   # K slabs add a reduction kernel
            _lib.ptr(out), _lib.ptr(a), _lib.ptr(b), _lib.ptr(bias), m, n, kd,
            a.stride(0), b.stride(0), out.stride(0), int(trans_a), int(trans_b),
            _lib.DTYPE_CODE[a.dtype], _lib.DTYPE_CODE[out.dtype], int(accumulate),
            _lib.ptr(ws), ws_bytes, _lib.current_stream_ptr(a.device))
    return out


def gemm_f32(a: Tensor, b: Tensor, trans_a: bool = False, trans_b: bool = False,
             col_bias: Optional[Tensor] = None, name: Optional[str] = None) -> Tensor:
    """C = op(a) @ op(b) for float32 CUDA matrices on the 16-bit tensor cores (``sru_b200_gemm_f32``: three-way
    bfloat16 split of both operands, six partial products in one GEMM, fp32 accumulation).  All three extents must
    be multiples of 8."""
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise _lib.SruB200Error("gemm_f32 operands must be float32")
    a = a if a.stride(1) == 1 else a.contiguous()
    b = b if b.stride(1) == 1 else b.contiguous()
    m = a.size(1) if trans_a else a.size(0)
    kd = a.size(0) if trans_a else a.size(1)
    n = b.size(0) if trans_b else b.size(1)
    out = torch.empty(m, n, dtype=torch.float32, device=a.device)
    if m == 0 or n == 0:
        return out
    bias = None if col_bias is None else col_bias.detach().float().contiguous()
    L = _lib.lib()
    with torch.cuda.device(a.device):
        ws_bytes = int(L.sru_b200_gemm_f32_workspace_bytes(m, n, kd))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
        if name is None:
            name = "gemm_wgrad" if trans_a else ("gemm_dgrad" if trans_b else "gemm_fwd")
        _lib.call(name, 3, L.sru_b200_gemm_f32, _lib.ptr(out), _lib.ptr(a), _lib.ptr(b), _lib.ptr(bias), m, n, kd,
                  a.stride(0), b.stride(0), out.stride(0), int(trans_a), int(trans_b), 0, _lib.ptr(ws), ws_bytes,
                  _lib.current_stream_ptr(a.device))
    return out


_fp32_tensor = False


def set_fp32_on_tensor_cores(flag: bool) -> None:
    """float32 projections on the tcgen05 GEMM through the three-way bfloat16 split, or (default) on the library's
    float32 GEMM (``torch.mm``).  Off by default because of accuracy: the tensor cores do not round their fp32
    accumulation like IEEE additions, and the measured error of the split product is 2e-6 of the largest element at
    K = 128 and 2e-5 at K = 2048 (library float32 GEMM: 5e-7 / 2e-6) -- above the 1e-5 parity bar for long
    reductions, and above the reference's own 1e-4 absolute test bound on gradients of magnitude ~100."""
    global _fp32_tensor
    _fp32_tensor = bool(flag)


def fp32_on_tensor_cores() -> bool:
    return _fp32_tensor


class _ProjectionF32(Function):
    """x (M, K) @ w (K, N), all float32, forward and both gradients through gemm_f32."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return gemm_f32(x, w)

    @staticmethod
    def backward(ctx, grad_u):
        x, w = ctx.saved_tensors
        grad_u = grad_u.contiguous().float()
        gx = gemm_f32(grad_u, w, trans_b=True) if ctx.needs_input_grad[0] else None
        gw = gemm_f32(x, grad_u, trans_a=True) if ctx.needs_input_grad[1] else None
        return gx, gw


_grad_link_on = True


def set_grad_link_enabled(flag: bool) -> None:
    """Switches the fused gradient sum of a layer input (GradLink) on or off; on by default.  Off, autograd
    adds the scan's and the GEMM's gradient of the input itself (one more pass over the tensor)."""
    global _grad_link_on
    _grad_link_on = bool(flag)


def grad_link_enabled() -> bool:
    return _grad_link_on


class GradLink:
    """Joins the two gradients of a layer input.

    A k = 3 layer uses its input twice: as the GEMM operand (U = x W) and as the highway term of
    the scan.  Autograd would materialise both gradients and add them with one more pass over
    (length, batch, width).  With a link, the scan's backward leaves its grad_x here instead of
    returning it, and the projection's backward, which always runs later (U feeds the scan),
    lets the dgrad GEMM accumulate onto that buffer in its epilogue and returns the sum.

    ``armed`` is set by project() when the tensor it was given goes into the GEMM as it is (same
    storage and dtype), i.e. when "gradient of the GEMM operand" and "gradient of x" are the same
    thing; the scan side only uses an armed link.
    """
    __slots__ = ("armed", "grad_x")

    def __init__(self):
        self.armed = False
        self.grad_x = None


class _Projection(Function):
    """x (M, K) in the 16-bit compute type times the MASTER weight w (K, N).  The weight is rounded to the compute
    type inside (what autocast does in front of ``mm``), but its gradient leaves the weight-gradient GEMM in the
    master's own type: with float32 parameters the fp32 accumulators are stored as they are, instead of being
    rounded to 16 bits and cast back (one pass less, and no overflow of a half-precision sum over length * batch
    rows under a loss scale)."""

    @staticmethod
    def forward(ctx, x, w, col_bias, link):
        dt = x.dtype
        wc = w.detach()
        if wc.dtype != dt:
            wc = wc.to(dt)
        if not wc.is_contiguous():
            wc = wc.contiguous()
        ctx.save_for_backward(x, wc)
        ctx.w_dtype = w.dtype if w.dtype in (torch.float32,) + _SIXTEEN else dt
        ctx.link = link
        return gemm(x, wc, col_bias=col_bias)

    @staticmethod
    def backward(ctx, grad_u):
        x, w = ctx.saved_tensors
        grad_u = grad_u.contiguous()
        gx = gw = None
        highway = None
        if ctx.link is not None:
            highway, ctx.link.grad_x = ctx.link.grad_x, None
        if ctx.needs_input_grad[0]:
            if highway is not None and highway.dtype == x.dtype and highway.numel() == x.numel() \
                    and highway.is_contiguous():
                # (M,N) x (K,N)^T added onto the scan's highway gradient in the epilogue
                gx = gemm(grad_u, w, trans_b=True, out=highway.view(x.shape), accumulate=True)
            else:
                gx = gemm(grad_u, w, trans_b=True)        # (M,N) x (K,N)^T -> (M,K)
                if highway is not None:
                    gx = gx + highway.reshape(gx.shape).to(gx.dtype)
        if ctx.needs_input_grad[1]:
            gw = gemm(x, grad_u, trans_a=True, out_dtype=ctx.w_dtype)     # (M,K)^T x (M,N) -> (K,N)
        return gx, gw, None, None


_bias_fold_on = True


def set_bias_fold_enabled(flag: bool) -> None:
    """Gate bias added to U by the projection GEMM's epilogue (and the scan called without bias): on by default
    for 16-bit projections on the tcgen05 kernel; off, the scan adds the bias itself."""
    global _bias_fold_on
    _bias_fold_on = bool(flag)


def bias_fold_enabled() -> bool:
    return _bias_fold_on


def gate_bias_columns(bias: Tensor, width: int, k: int) -> Tensor:
    """The layer's bias (2 * width,) laid out as float[width * k] for U's gate-innermost columns
    (``sru_b200_gate_bias_columns``).  No gradient flows through it: grad_bias comes from the backward scan."""
    b = bias.detach()
    if b.dtype != torch.float32 or not b.is_contiguous():
        b = b.float().contiguous()
    out = torch.empty(width * k, dtype=torch.float32, device=b.device)
    with torch.cuda.device(b.device):
        _lib.call("gate_bias", 1, _lib.lib().sru_b200_gate_bias_columns, _lib.ptr(out), _lib.ptr(b), width, k,
                  _lib.current_stream_ptr(b.device))
    return out


def _native_operand(x: Tensor, w: Tensor):
    """The compute type of this product and x in that type, if the tcgen05 kernel takes it; else (None, None)."""
    dt = x.dtype
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
    elif w.dtype != x.dtype:
        dt = w.dtype
    if dt not in _SIXTEEN or gemm_backend() != "tcgen05":
        return dt, None
    xc = x if x.dtype == dt else x.to(dt)
    xc = xc if xc.is_contiguous() else xc.contiguous()
    if not (xc.size(1) % 8 == 0 and w.size(1) % 8 == 0 and xc.size(0) % 8 == 0 and xc.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and w.is_contiguous()):
        return dt, None      # the tensor-map loads need 16-byte aligned bases and row pitches
    return dt, xc


def will_run_native(x: Tensor, w: Tensor) -> bool:
    """True if project(x, w) would run on the tcgen05 kernel (16-bit compute type, aligned shapes)."""
    return x.is_cuda and _native_operand(x, w)[1] is not None


def project(x: Tensor, w: Tensor, col_bias: Optional[Tensor] = None,
            link: Optional[GradLink] = None) -> Tensor:
    """x (M, K) @ w (K, N) (+ col_bias) with autograd.  Follows autocast: inside an autocast region the
    operands are rounded to the autocast dtype, as ``Tensor.mm`` would.  ``link`` (see GradLink)
    is armed when x itself becomes the GEMM operand and x needs a gradient.  ``col_bias`` is a constant here
    (no gradient)."""
    if not x.is_cuda:
        raise _lib.SruB200Error("sru_b200 has no CPU path: the projection input must be a CUDA tensor")
    dt, xc = _native_operand(x, w)
    if xc is not None:
        if link is not None:
            link.armed = xc is x and x.requires_grad and torch.is_grad_enabled()
        with torch.autocast("cuda", enabled=False):
            return _Projection.apply(xc, w, col_bias, link if link is not None and link.armed else None)
    if (_fp32_tensor and gemm_backend() == "tcgen05" and x.dtype == torch.float32 and w.dtype == torch.float32
            and not torch.is_autocast_enabled("cuda") and x.dim() == 2 and x.size(0) % 8 == 0 and x.size(1) % 8 == 0
            and w.size(1) % 8 == 0 and x.size(0) > 0):
        out = _ProjectionF32.apply(x.contiguous(), w.contiguous())
    else:
        out = x.mm(w) if x.dtype == w.dtype or torch.is_autocast_enabled("cuda") else x.to(dt).mm(w)
    if col_bias is not None:
        out = out + col_bias.to(out.dtype)
    return out
