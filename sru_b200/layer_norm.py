"""Layer normalisation of the SRU layer (``nn.LayerNorm`` at sru/modules.py:155-160, applied at
:252-253 before the projection or at :278-279 after the recurrence) on this package's kernels
(``sru_b200_layer_norm_forward`` / ``_backward`` of the C ABI).

``layer_norm(x, weight, bias, eps, out_dtype)`` normalises the last dimension.  With fp32 input
and a 16-bit ``out_dtype`` the normalised rows are written directly in the type the projection
GEMM consumes: the separate cast pass that autocast inserts between ``layer_norm`` (fp32) and
``mm`` (16-bit) disappears, the values are the same (one rounding of the fp32 result).

Row lengths the kernels do not take (not a multiple of 8 / 4 elements, or above 4096) go to the
library operator ``torch.nn.functional.layer_norm``; everything else raises if the native
library is missing.
"""
from typing import Optional

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.autograd import Function

from . import _lib

_SIXTEEN = (torch.float16, torch.bfloat16)
MAX_ROW = 4096


def supported(x: Tensor, out_dtype: torch.dtype) -> bool:
    """True if the native kernels take this row length and type combination."""
    n = x.size(-1)
    if x.dtype == torch.float32:
        ok_types = out_dtype in (torch.float32,) + _SIXTEEN
        gran = 4
    elif x.dtype in _SIXTEEN:
        ok_types = out_dtype == x.dtype
        gran = 8
    else:
        return False
    return ok_types and n % gran == 0 and 0 < n <= MAX_ROW


def forward_raw(x2d: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], eps: float,
                out_dtype: torch.dtype, need_stats: bool = True):
    """x2d (rows, n) contiguous -> (y, mean, rstd); mean / rstd are None without need_stats."""
    rows, n = x2d.shape
    y = torch.empty(rows, n, dtype=out_dtype, device=x2d.device)
    mean = torch.empty(rows, dtype=torch.float32, device=x2d.device) if need_stats else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x2d.device) if need_stats else None
    if rows == 0:
        return y, mean, rstd
    w = None if weight is None else weight.detach().float().contiguous()
    b = None if bias is None else bias.detach().float().contiguous()
    L = _lib.lib()
    with torch.cuda.device(x2d.device):
        _lib.call("layer_norm_fwd", 1, L.sru_b200_layer_norm_forward,
                  _lib.ptr(y), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(x2d), _lib.ptr(w), _lib.ptr(b),
                  rows, n, float(eps), _lib.DTYPE_CODE[x2d.dtype], _lib.DTYPE_CODE[out_dtype],
                  _lib.current_stream_ptr(x2d.device))
    return y, mean, rstd


def backward_raw(dy2d: Tensor, x2d: Tensor, mean: Tensor, rstd: Tensor, weight: Optional[Tensor],
                 need_wb: bool = True):
    """-> (dx in x's dtype, dgamma fp32, dbeta fp32); the last two are None without need_wb."""
    rows, n = x2d.shape
    dx = torch.empty_like(x2d)
    dg = torch.empty(n, dtype=torch.float32, device=x2d.device) if need_wb else None
    db = torch.empty(n, dtype=torch.float32, device=x2d.device) if need_wb else None
    w = None if weight is None else weight.detach().float().contiguous()
    L = _lib.lib()
    with torch.cuda.device(x2d.device):
        ws_bytes = int(L.sru_b200_layer_norm_backward_workspace_bytes(rows, n))
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x2d.device)
        _lib.call("layer_norm_bwd", 2 if need_wb else 1, L.sru_b200_layer_norm_backward,
                  _lib.ptr(dx), _lib.ptr(dg), _lib.ptr(db), _lib.ptr(dy2d), _lib.ptr(x2d), _lib.ptr(mean),
                  _lib.ptr(rstd), _lib.ptr(w), rows, n, _lib.DTYPE_CODE[x2d.dtype],
                  _lib.DTYPE_CODE[dy2d.dtype], _lib.ptr(ws), ws_bytes, _lib.current_stream_ptr(x2d.device))
    return dx, dg, db


class _LayerNorm(Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_dtype):
        x2d = x.detach().contiguous().view(-1, x.size(-1))
        need = any(ctx.needs_input_grad[:3])
        y, mean, rstd = forward_raw(x2d, weight, bias, eps, out_dtype, need_stats=need)
        ctx.save_for_backward(x2d, mean, rstd, weight)
        ctx.x_shape = x.shape
        ctx.param_dtypes = (None if weight is None else weight.dtype, None if bias is None else bias.dtype)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2d, mean, rstd, weight = ctx.saved_tensors
        out_dtype = dy.dtype
        dy2d = dy.contiguous().view(x2d.shape)
        need_wb = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        dx, dg, db = backward_raw(dy2d, x2d, mean, rstd, weight, need_wb=need_wb)
        wdt, bdt = ctx.param_dtypes
        gx = dx.view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        gw = dg.to(wdt) if (ctx.needs_input_grad[1] and wdt is not None) else None
        gb = db.to(bdt) if (ctx.needs_input_grad[2] and bdt is not None) else None
        return gx, gw, gb, None, None


def layer_norm(x: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], eps: float = 1e-5,
               out_dtype: Optional[torch.dtype] = None) -> Tensor:
    """LayerNorm over the last dimension of a CUDA tensor, with autograd.

    out_dtype None: what the reference's call returns — float32 inside an autocast region
    (autocast runs layer_norm in float32), x's dtype otherwise.
    """
    if not x.is_cuda:
        raise _lib.SruB200Error("sru_b200 has no CPU path: layer_norm input must be a CUDA tensor")
    if out_dtype is None:
        out_dtype = torch.float32 if torch.is_autocast_enabled("cuda") else x.dtype
    xin = x
    if xin.dtype in _SIXTEEN and out_dtype != xin.dtype:
        xin = xin.float()          # 16-bit in, other type out: normalise in fp32 like autocast does
    if not supported(xin, out_dtype):
        with torch.autocast("cuda", enabled=False):
            y = F.layer_norm(xin.float(), (x.size(-1),), None if weight is None else weight.float(),
                             None if bias is None else bias.float(), eps)
        return y.to(out_dtype)
    with torch.autocast("cuda", enabled=False):
        return _LayerNorm.apply(xin, weight, bias, eps, out_dtype)
