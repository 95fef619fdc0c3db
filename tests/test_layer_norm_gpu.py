"""Layer-normalisation kernels (C ABI sru_b200_layer_norm_forward / _backward) against the CPU oracle and the
golden vectors taken from the reference's nn.LayerNorm.

Tolerances: fp32 rows 1e-5 relative (max-abs error over max-abs reference, per tensor); 16-bit outputs add one
rounding of the result (bf16 2^-9, fp16 2^-11): bound 1e-2.  The 16-bit comparisons feed the oracle the same
16-bit-rounded inputs.
"""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ln():
    from sru_b200 import layer_norm
    return layer_norm


def _oracle():
    from oracle import sru_oracle
    return sru_oracle


def test_golden_vectors_fp32(layer_norm_cases):
    """fp32 kernels on the reference's float64 vectors: y, dx, dweight, dbias within 1e-5."""
    ln = _ln()
    for case in layer_norm_cases:
        n = case["n"]
        x = case["x"].float().reshape(-1, n).to(DEV)
        w, b = case["weight"].float().to(DEV), case["bias"].float().to(DEV)
        dy = case["dy"].float().reshape(-1, n).to(DEV)
        y, mean, rstd = ln.forward_raw(x, w, b, case["eps"], torch.float32)
        dx, dg, db = ln.backward_raw(dy, x, mean, rstd, w)
        assert rel_err(y.view_as(case["y"]), case["y"]) <= 1e-5, n
        assert rel_err(dx.view_as(case["dx"]), case["dx"]) <= 1e-5, n
        assert rel_err(dg, case["dweight"]) <= 1e-5, n
        assert rel_err(db, case["dbias"]) <= 1e-5, n


COMBOS = [
    (torch.float32, torch.float32, 1e-5, 1e-5),
    (torch.float32, torch.bfloat16, 1e-2, 1e-5),
    (torch.float32, torch.float16, 2e-3, 1e-5),
    (torch.bfloat16, torch.bfloat16, 1e-2, 1e-2),
    (torch.float16, torch.float16, 2e-3, 2e-3),
]


@pytest.mark.parametrize("rows,n", [(1, 8), (3, 120), (130, 512), (1000, 1024), (257, 2048), (66, 4096),
                                     (5, 24), (4099, 256), (7, 3072)])
@pytest.mark.parametrize("x_dtype,y_dtype,tol_y,tol_dx", COMBOS)
def test_kernels_vs_oracle(rows, n, x_dtype, y_dtype, tol_y, tol_dx):
    """Every type pair and warps-per-row variant, ragged row counts, more rows than one wave of CTAs."""
    ln, oracle = _ln(), _oracle()
    g = torch.Generator().manual_seed(rows * 7 + n)
    x = (torch.randn(rows, n, generator=g) * 1.5 + 0.3).to(x_dtype)
    w = torch.randn(n, generator=g) * 0.5 + 1.0
    b = torch.randn(n, generator=g) * 0.2
    dy = torch.randn(rows, n, generator=g).to(y_dtype)
    # oracle in float64 on the rounded inputs
    ry, rmean, rrstd = oracle.layer_norm_forward(x.double(), w.double(), b.double(), 1e-5)
    rdx, rdg, rdb = oracle.layer_norm_backward(dy.double(), x.double(), rmean, rrstd, w.double())
    y, mean, rstd = ln.forward_raw(x.to(DEV), w.to(DEV), b.to(DEV), 1e-5, y_dtype)
    dx, dg, db = ln.backward_raw(dy.to(DEV), x.to(DEV), mean, rstd, w.to(DEV))
    torch.cuda.synchronize()
    assert y.dtype == y_dtype and dx.dtype == x_dtype and dg.dtype == torch.float32
    assert rel_err(mean, rmean) <= 1e-5 and rel_err(rstd, rrstd) <= 1e-5
    assert rel_err(y, ry) <= tol_y, rel_err(y, ry)
    assert rel_err(dx, rdx) <= tol_dx, rel_err(dx, rdx)
    # the column sums see fp32 data whatever the storage types are: only the rounding of mean / rstd enters
    assert rel_err(dg, rdg) <= 2e-5 and rel_err(db, rdb) <= 2e-5, (rel_err(dg, rdg), rel_err(db, rdb))


def test_no_affine_and_no_stats():
    ln, oracle = _ln(), _oracle()
    g = torch.Generator().manual_seed(3)
    x = torch.randn(50, 256, generator=g)
    ry, rmean, rrstd = oracle.layer_norm_forward(x.double(), None, None, 1e-5)
    y, mean, rstd = ln.forward_raw(x.to(DEV), None, None, 1e-5, torch.float32, need_stats=False)
    assert mean is None and rstd is None and rel_err(y, ry) <= 1e-5
    y2, mean, rstd = ln.forward_raw(x.to(DEV), None, None, 1e-5, torch.float32)
    dy = torch.randn(50, 256, generator=g)
    rdx, _, _ = oracle.layer_norm_backward(dy.double(), x.double(), rmean, rrstd, None)
    dx, dg, db = ln.backward_raw(dy.to(DEV), x.to(DEV), mean, rstd, None, need_wb=False)
    assert dg is None and db is None and rel_err(dx, rdx) <= 1e-5


def test_backward_is_deterministic():
    """Column sums are combined in a fixed order: repeated calls give identical bits."""
    ln = _ln()
    g = torch.Generator().manual_seed(4)
    x = torch.randn(20000, 512, generator=g).to(DEV)
    w = torch.randn(512, generator=g).to(DEV)
    dy = torch.randn(20000, 512, generator=g).to(DEV)
    _, mean, rstd = ln.forward_raw(x, w, None, 1e-5, torch.float32)
    a = ln.backward_raw(dy, x, mean, rstd, w)
    b = ln.backward_raw(dy, x, mean, rstd, w)
    assert all(torch.equal(p, q) for p, q in zip(a, b))


def test_autograd_function_and_autocast_types():
    """layer_norm(): autograd gradients equal the oracle's; inside autocast the default output is float32
    (as the reference's call), and an explicit 16-bit output equals the rounded float32 result."""
    ln, oracle = _ln(), _oracle()
    g = torch.Generator().manual_seed(6)
    x0 = torch.randn(6, 11, 256, generator=g)
    w0 = torch.randn(256, generator=g) * 0.4 + 1
    b0 = torch.randn(256, generator=g) * 0.1
    xr, wr, br = (t.double().requires_grad_(True) for t in (x0, w0, b0))
    yr = oracle.layer_norm_oracle(xr, wr, br, 1e-5)
    (yr * yr).sum().backward()
    x, w, b = (t.to(DEV).requires_grad_(True) for t in (x0, w0, b0))
    y = ln.layer_norm(x, w, b, 1e-5)
    (y * y).sum().backward()
    assert y.shape == x.shape and y.dtype == torch.float32
    for got, ref in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad), (b.grad, br.grad)):
        assert rel_err(got, ref) <= 1e-5
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y32 = ln.layer_norm(x, w, b, 1e-5)
        y16 = ln.layer_norm(x, w, b, 1e-5, out_dtype=torch.bfloat16)
    assert y32.dtype == torch.float32 and y16.dtype == torch.bfloat16
    assert torch.equal(y16, y32.bfloat16())


def test_unsupported_rows_use_the_library_operator():
    """Row lengths outside the kernels' range (not a multiple of 4, above 4096) still work through layer_norm()."""
    ln, oracle = _ln(), _oracle()
    for n in (2, 30, 4100):
        g = torch.Generator().manual_seed(n)
        x = torch.randn(9, n, generator=g)
        w, b = torch.randn(n, generator=g), torch.randn(n, generator=g)
        ry, _, _ = oracle.layer_norm_forward(x.double(), w.double(), b.double(), 1e-5)
        y = ln.layer_norm(x.to(DEV), w.to(DEV), b.to(DEV), 1e-5)
        assert rel_err(y, ry) <= 1e-5, n


def test_bad_arguments_are_reported():
    from sru_b200 import _lib
    L = _lib.lib()
    x = torch.zeros(4, 16, device=DEV)
    rc = L.sru_b200_layer_norm_forward(x.data_ptr(), None, None, x.data_ptr(), None, None, 4, 18, 1e-5, 0, 0, None)
    assert rc == -2 and b"multiple" in L.sru_b200_last_error()
    rc = L.sru_b200_layer_norm_forward(x.data_ptr(), None, None, x.data_ptr(), None, None, 4, 16, 1e-5, 2, 0, None)
    assert rc == -2
    rc = L.sru_b200_layer_norm_forward(None, None, None, None, None, None, 4, 16, 1e-5, 0, 0, None)
    assert rc == -1
    rc = L.sru_b200_layer_norm_backward(x.data_ptr(), None, None, x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                        x.data_ptr(), None, 4, 16, 0, 0, None, 0, None)
    assert rc == -3 and b"workspace" in L.sru_b200_last_error()
    with pytest.raises(_lib.SruB200Error):
        _ln().layer_norm(torch.zeros(2, 8), None, None)
