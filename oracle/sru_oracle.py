"""ctypes front end of the CPU oracle (``sru_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline legs import this
module; the shipped package never does.

``elementwise_recurrence_oracle`` has the call signature of the reference's
``sru.ops.elementwise_recurrence_naive`` (sru/ops.py:146-157) and is differentiable:
its backward is the C restatement of the reference's CUDA adjoint
(sru/csrc/sru_cuda_kernel.cu:447-578, :667-822), not autograd through a Python loop.
"""
import ctypes
import os
from typing import Optional

import torch

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build_oracle())
    return _lib


def set_threads(n: int):
    """Pin the OpenMP thread count used by the oracle loops (columns are independent)."""
    try:
        omp = ctypes.CDLL("libgomp.so.1")
        omp.omp_set_num_threads(int(n))
    except OSError:
        pass


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _suffix_and_real(dtype):
    if dtype == torch.float32:
        return "_f32", ctypes.c_float
    if dtype == torch.float64:
        return "_f64", ctypes.c_double
    raise TypeError("oracle computes in float32 or float64, got %s" % dtype)


def _prep(t, dtype):
    return None if t is None else t.detach().to(dtype).contiguous()


def forward(u, x, weight_c, bias, c_init, mask_c, mask_pad, L, B, d, dirs, k,
            activation_type, skip_type, is_custom, scale_x=1.0):
    """Returns (h (L,B,D), c_hist (L,B,D), c_last (B,D)) on CPU in u's dtype."""
    dtype = u.dtype
    sfx, real = _suffix_and_real(dtype)
    D = d * dirs
    u = _prep(u, dtype)
    x = _prep(x, dtype) if skip_type == 1 else None
    weight_c, bias = _prep(weight_c, dtype), _prep(bias, dtype)
    c_init, mask_c = _prep(c_init, dtype), _prep(mask_c, dtype)
    pad = None if mask_pad is None else (mask_pad != 0).to(torch.uint8).contiguous()
    h = torch.empty(L, B, D, dtype=dtype)
    c_hist = torch.empty(L, B, D, dtype=dtype)
    c_last = torch.empty(B, D, dtype=dtype)
    fn = getattr(lib(), "sru_oracle_forward" + sfx)
    fn.restype = None
    fn(_p(h), _p(c_hist), _p(c_last), _p(u), _p(x), _p(weight_c), _p(bias), _p(c_init),
       _p(mask_c), _p(pad), ctypes.c_long(L), ctypes.c_long(B), ctypes.c_long(d),
       ctypes.c_int(dirs), ctypes.c_int(k), ctypes.c_int(activation_type),
       ctypes.c_int(skip_type), ctypes.c_int(int(is_custom)), real(float(scale_x)))
    return h, c_hist, c_last


def backward(u, x, weight_c, bias, c_init, mask_c, mask_pad, c_hist, grad_h, grad_last,
             L, B, d, dirs, k, activation_type, skip_type, is_custom, scale_x=1.0):
    """Returns (grad_u, grad_x or None, grad_wc, grad_bias (2D,), grad_init (B,D))."""
    dtype = u.dtype
    sfx, real = _suffix_and_real(dtype)
    D = d * dirs
    u = _prep(u, dtype)
    x = _prep(x, dtype) if skip_type == 1 else None
    weight_c, bias = _prep(weight_c, dtype), _prep(bias, dtype)
    c_init, mask_c = _prep(c_init, dtype), _prep(mask_c, dtype)
    c_hist, grad_h = _prep(c_hist, dtype), _prep(grad_h, dtype)
    grad_last = _prep(grad_last, dtype)
    pad = None if mask_pad is None else (mask_pad != 0).to(torch.uint8).contiguous()
    grad_u = torch.empty(L, B, D * k, dtype=dtype)
    grad_x = torch.empty(L, B, D, dtype=dtype) if skip_type == 1 else None
    grad_wc = torch.empty(L, B, D * 2, dtype=dtype) if is_custom else torch.empty(2 * D, dtype=dtype)
    grad_bias = torch.empty(2 * D, dtype=dtype)
    grad_init = torch.empty(B, D, dtype=dtype)
    fn = getattr(lib(), "sru_oracle_backward" + sfx)
    fn.restype = None
    fn(_p(grad_u), _p(grad_x), _p(grad_wc), _p(grad_bias), _p(grad_init),
       _p(u), _p(x), _p(weight_c), _p(bias), _p(c_init), _p(mask_c), _p(pad),
       _p(c_hist), _p(grad_h), _p(grad_last),
       ctypes.c_long(L), ctypes.c_long(B), ctypes.c_long(d),
       ctypes.c_int(dirs), ctypes.c_int(k), ctypes.c_int(activation_type),
       ctypes.c_int(skip_type), ctypes.c_int(int(is_custom)), real(float(scale_x)))
    return grad_u, grad_x, grad_wc, grad_bias, grad_init


class _OracleRecurrence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, x, weight_c, bias, c_init, mask_c, mask_pad, meta):
        L, B, d, dirs, k, act, skip, custom, scale = meta
        h, c_hist, c_last = forward(u, x, weight_c, bias, c_init, mask_c, mask_pad,
                                    L, B, d, dirs, k, act, skip, custom, scale)
        ctx.meta = meta
        ctx.mask_pad = mask_pad
        ctx.x_shape = None if x is None else x.shape
        ctx.save_for_backward(u, x if skip == 1 else None, weight_c, bias, c_init, mask_c, c_hist)
        return h, c_last

    @staticmethod
    def backward(ctx, grad_h, grad_last):
        u, x, weight_c, bias, c_init, mask_c, c_hist = ctx.saved_tensors
        L, B, d, dirs, k, act, skip, custom, scale = ctx.meta
        gu, gx, gwc, gb, gi = backward(u, x, weight_c, bias, c_init, mask_c, ctx.mask_pad,
                                       c_hist, grad_h, grad_last,
                                       L, B, d, dirs, k, act, skip, custom, scale)
        gu = gu.view_as(u)
        if gx is not None:
            gx = gx.view(ctx.x_shape)
        gwc = gwc.view_as(weight_c)
        gi = gi.view_as(c_init)
        return gu, gx, gwc, gb.view_as(bias), gi, None, None, None


def elementwise_recurrence_oracle(U, x, weight_c, bias, c_init, activation_type: int,
                                  hidden_size: int, bidirectional: bool, has_skip_term: bool,
                                  scale_x=None, dropout_mask_c=None, mask_pad=None):
    """Same arguments and return value as sru/ops.py:146 elementwise_recurrence_naive."""
    dirs = 2 if bidirectional else 1
    L = x.size(0) if x.dim() == 3 else 1
    B = x.size(-2)
    d = hidden_size
    k = U.size(-1) // d // dirs
    is_custom = weight_c.dim() > 1
    skip = 0 if not has_skip_term else (1 if k == 3 else 2)
    scale = 1.0 if scale_x is None else float(scale_x.reshape(-1)[0])
    meta = (L, B, d, dirs, k, int(activation_type), skip, is_custom, scale)
    dt = U.dtype
    h, c_last = _OracleRecurrence.apply(
        U.contiguous(), x.to(dt).contiguous(), weight_c.to(dt).contiguous(), bias.to(dt),
        c_init.to(dt).contiguous(),
        None if dropout_mask_c is None else dropout_mask_c.to(dt).contiguous(),
        mask_pad, meta)
    if x.dim() == 2:
        h = h.squeeze(0)
    return h, c_last


def layer_norm_forward(x2d, gamma, beta, eps):
    """(rows, n) -> (y, mean, rstd) on CPU in x2d's dtype (float32 or float64)."""
    dtype = x2d.dtype
    sfx, _ = _suffix_and_real(dtype)
    x2d = _prep(x2d, dtype)
    gamma, beta = _prep(gamma, dtype), _prep(beta, dtype)
    rows, n = x2d.shape
    y = torch.empty_like(x2d)
    mean = torch.empty(rows, dtype=dtype)
    rstd = torch.empty(rows, dtype=dtype)
    getattr(lib(), "sru_oracle_layer_norm_forward" + sfx)(
        _p(y), _p(mean), _p(rstd), _p(x2d), _p(gamma), _p(beta),
        ctypes.c_long(rows), ctypes.c_long(n), ctypes.c_double(float(eps)))
    return y, mean, rstd


def layer_norm_backward(dy2d, x2d, mean, rstd, gamma):
    """-> (dx, dgamma, dbeta) on CPU in x2d's dtype."""
    dtype = x2d.dtype
    sfx, _ = _suffix_and_real(dtype)
    x2d, dy2d = _prep(x2d, dtype), _prep(dy2d, dtype)
    mean, rstd, gamma = _prep(mean, dtype), _prep(rstd, dtype), _prep(gamma, dtype)
    rows, n = x2d.shape
    dx = torch.empty_like(x2d)
    dg = torch.empty(n, dtype=dtype)
    db = torch.empty(n, dtype=dtype)
    getattr(lib(), "sru_oracle_layer_norm_backward" + sfx)(
        _p(dx), _p(dg), _p(db), _p(dy2d), _p(x2d), _p(mean), _p(rstd), _p(gamma),
        ctypes.c_long(rows), ctypes.c_long(n))
    return dx, dg, db


class _OracleLayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        x2d = x.detach().contiguous().view(-1, x.size(-1))
        y, mean, rstd = layer_norm_forward(x2d, gamma, beta, eps)
        ctx.save_for_backward(x2d, mean, rstd, gamma)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2d, mean, rstd, gamma = ctx.saved_tensors
        dx, dg, db = layer_norm_backward(dy.contiguous().view(x2d.shape), x2d, mean, rstd, gamma)
        return dx.view(ctx.shape), dg, db, None


def layer_norm_oracle(x, gamma, beta, eps=1e-5):
    """Differentiable CPU layer norm over the last dimension (float32 or float64 tensors)."""
    dt = x.dtype
    return _OracleLayerNorm.apply(x, gamma.to(dt), beta.to(dt), eps)
