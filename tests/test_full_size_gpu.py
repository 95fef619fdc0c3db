"""The kernels at the full sizes of the benchmark configurations, checked through properties that do not need a
full-size CPU run:

* columns of different batch rows are independent, so a few batch rows of the full-size GPU result are compared
  with the CPU oracle run on just those rows (2e-2 for 16-bit storage, as everywhere);
* the batch-reduced parameter gradients are additive over disjoint batch chunks (sum of the chunk results equals
  the full result);
* sampled rows of the full-size GEMM are compared with an fp32 matmul of those rows.

Inputs are generated on the device (the tensors are GBs); scale 0.5 keeps gates away from saturation.
"""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from sru_b200 import ops
    return ops


def _oracle():
    from oracle import sru_oracle
    return sru_oracle


def _device_inputs(L, B, d, dirs, k, dtype, pad, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    D = d * dirs
    U = (torch.randn(L, B, D * k, device=DEV, generator=g) * 0.5).to(dtype)
    x = (torch.randn(L, B, D, device=DEV, generator=g) * 0.5).to(dtype)
    wc = torch.randn(2 * D, device=DEV, generator=g) * 0.5
    bias = torch.randn(2 * D, device=DEV, generator=g) * 0.5
    c0 = torch.randn(B, D, device=DEV, generator=g) * 0.5
    mc = (torch.rand(B, D, device=DEV, generator=g) > 0.1).float() / 0.9
    mp = None
    if pad:
        lens = torch.randint(int(L * 0.6), L + 1, (B,), device=DEV, generator=g)
        mp = (torch.arange(L, device=DEV).view(L, 1) >= lens.view(1, B)).contiguous()
    gh = (torch.randn(L, B, D, device=DEV, generator=g) * 0.5).to(dtype)
    gl = torch.randn(B, D, device=DEV, generator=g) * 0.5
    return U, x, wc, bias, c0, mc, mp, gh, gl


def _oracle_rows(rows, U, x, wc, bias, c0, mc, mp, gh, gl, L, d, dirs, k, need_grad):
    """CPU oracle (fp32) on the batch rows `rows` of the device tensors."""
    oracle = _oracle()
    f = lambda t: None if t is None else t[:, rows].float().cpu().contiguous()
    f2 = lambda t: None if t is None else t[rows].float().cpu().contiguous()
    Us, xs, ghs = f(U), f(x), f(gh)
    mps = None if mp is None else mp[:, rows].cpu().contiguous()
    nb = len(rows)
    skip = 1 if k == 3 else 2
    h, ch, cl = oracle.forward(Us, xs, wc.cpu(), bias.cpu(), f2(c0), f2(mc), mps, L, nb, d, dirs, k, 0, skip, False, 1.0)
    out = dict(h=h, c_last=cl)
    if need_grad:
        gu, gx, gwc, gb, gi = oracle.backward(Us, xs, wc.cpu(), bias.cpu(), f2(c0), f2(mc), mps, ch, ghs, f2(gl),
                                              L, nb, d, dirs, k, 0, skip, False, 1.0)
        out.update(grad_u=gu, grad_x=gx, grad_init=gi)
    return out


def test_config5_layer_full_size():
    """One layer of configuration 5 (L=1000, B=256, bi 1024/dir, k=3, bf16, fp32 history, mask_pad, dropout mask)."""
    ops = _ops()
    L, B, d, dirs, k = 1000, 256, 1024, 2, 3
    U, x, wc, bias, c0, mc, mp, gh, gl = _device_inputs(L, B, d, dirs, k, torch.bfloat16, True, 55)
    h, c_hist, c_last = ops.scan_forward(U, x, wc, bias, c0, mc, mp, L, B, d, dirs, k, 0, 1, 0, 1.0, True)
    gu, gx, gwc, gb, gi = ops.scan_backward(U, x, wc, bias, c0, mc, mp, c_hist, gh, gl, L, B, d, dirs, k, 0, 1, 0, 1.0)
    torch.cuda.synchronize()
    from sru_b200 import _lib
    _lib.check_device_error()
    rows = [0, 97, 255]
    ref = _oracle_rows(rows, U, x, wc, bias, c0, mc, mp, gh, gl, L, d, dirs, k, True)
    D = d * dirs
    assert rel_err(h[:, rows], ref["h"].view(L, 3, D)) <= 2e-2
    assert rel_err(c_last[rows], ref["c_last"].view(3, D)) <= 2e-2
    assert rel_err(gu[:, rows], ref["grad_u"].view(L, 3, D * k)) <= 2e-2
    assert rel_err(gx[:, rows], ref["grad_x"].view(L, 3, D)) <= 2e-2
    assert rel_err(gi[rows], ref["grad_init"].view(3, D)) <= 2e-2
    # padded positions: h is zero, grad_u is zero
    padded = mp.unsqueeze(-1)
    assert float((h * padded).abs().max()) == 0.0 and float((gu * padded).abs().max()) == 0.0
    # additivity of the batch-reduced gradients over two halves of the batch
    parts = []
    for lo, hi in ((0, 128), (128, 256)):
        s = slice(lo, hi)
        sub = [t[:, s].contiguous() for t in (U, x)]
        ch = c_hist[:, s].contiguous()
        r = ops.scan_backward(sub[0], sub[1], wc, bias, c0[s].contiguous(), mc[s].contiguous(), mp[:, s].contiguous(),
                              ch, gh[:, s].contiguous(), gl[s].contiguous(), L, hi - lo, d, dirs, k, 0, 1, 0, 1.0)
        parts.append((r[2], r[3]))
        assert torch.equal(r[0], gu[:, s]) or rel_err(r[0], gu[:, s]) <= 1e-6      # per-position results do not depend on the batch
    assert rel_err(parts[0][0] + parts[1][0], gwc) <= 1e-4
    assert rel_err(parts[0][1] + parts[1][1], gb) <= 1e-4


def test_config4_full_size_inference():
    """Configuration 4 (L=8192, B=16, uni 1024, k=3, bf16, no history): h and the final state of two batch rows."""
    ops = _ops()
    L, B, d, dirs, k = 8192, 16, 1024, 1, 3
    U, x, wc, bias, c0, _, _, _, _ = _device_inputs(L, B, d, dirs, k, torch.bfloat16, False, 44)
    h, c_hist, c_last = ops.scan_forward(U, x, wc, bias, c0, None, None, L, B, d, dirs, k, 0, 1, 0, 1.0, False)
    torch.cuda.synchronize()
    assert c_hist is None
    rows = [3, 15]
    ref = _oracle_rows(rows, U, x, wc, bias, c0, None, None, None, None, L, d, dirs, k, False)
    assert rel_err(h[:, rows], ref["h"].view(L, 2, d)) <= 2e-2
    assert rel_err(c_last[rows], ref["c_last"].view(2, d)) <= 2e-2


@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
def test_config5_gemm_full_size(layout):
    """The three products of a 2048 -> 6144 layer at M = 256 000 (forward, dgrad, wgrad): sampled output rows."""
    from sru_b200.projection import gemm
    g = torch.Generator(device=DEV).manual_seed(9)
    M, N, K = 256000, 6144, 2048
    if layout == "nn":      # U = x W
        a = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
        b = (torch.randn(K, N, device=DEV, generator=g) * 0.05).bfloat16()
        out = gemm(a, b)
        rows = torch.tensor([0, 1, 127, 128, 65537, 255999], device=DEV)
        ref = a[rows].float() @ b.float()
        got = out[rows]
    elif layout == "nt":    # grad_x = grad_U W^T
        a = (torch.randn(M, N, device=DEV, generator=g) * 0.5).bfloat16()
        b = (torch.randn(K, N, device=DEV, generator=g) * 0.05).bfloat16()
        out = gemm(a, b, trans_b=True)
        rows = torch.tensor([0, 255, 256, 131071, 255999], device=DEV)
        ref = a[rows].float() @ b.float().t()
        got = out[rows]
    else:                   # grad_W = x^T grad_U : reduction over M
        a = (torch.randn(M, K, device=DEV, generator=g) * 0.1).bfloat16()
        b = (torch.randn(M, N, device=DEV, generator=g) * 0.1).bfloat16()
        out = gemm(a, b, trans_a=True, out_dtype=torch.float32)
        rows = torch.tensor([0, 129, 2047], device=DEV)
        ref = a[:, rows].float().t() @ b.float()
        got = out[rows]
    torch.cuda.synchronize()
    assert rel_err(got, ref) <= (1e-2 if layout != "tn" else 1e-3), rel_err(got, ref)
