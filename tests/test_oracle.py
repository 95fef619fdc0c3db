"""The CPU oracle against the golden vectors produced by the reference implementation."""
import os

import pytest
import torch

from conftest import rel_err
from oracle import sru_oracle
from oracle import build as oracle_build


def _run_case(case, dtype):
    m = case["meta"]
    dirs = m["dirs"]
    U = case["U"].detach().clone().to(dtype).requires_grad_(True)
    x = case["x"].detach().clone().to(dtype).requires_grad_(True)
    wc = case["weight_c"].detach().clone().to(dtype).requires_grad_(True)
    bias = case["bias"].detach().clone().to(dtype).requires_grad_(True)
    c0 = case["c_init"].detach().clone().to(dtype).requires_grad_(True)
    mc = None if case["mask_c"] is None else case["mask_c"].to(dtype)
    sx = None if m["scale"] is None else torch.tensor([m["scale"]], dtype=dtype)
    h, c_last = sru_oracle.elementwise_recurrence_oracle(
        U, x, wc, bias, c0, m["act"], m["d"], dirs == 2, m["has_skip"], sx, mc, case["mask_pad"])
    loss = (h * case["grad_h"].to(dtype)).sum() + (c_last * case["grad_last"].to(dtype)).sum()
    loss.backward()
    return dict(h=h, c_last=c_last, grad_U=U.grad, grad_x=x.grad, grad_weight_c=wc.grad,
                grad_bias=bias.grad, grad_c_init=c0.grad)


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-12), (torch.float32, 1e-5)])
def test_oracle_matches_reference_naive(op_cases, dtype, tol):
    for case in op_cases:
        out = _run_case(case, dtype)
        for key, val in out.items():
            ref = case[key]
            if ref is None:
                continue
            e = rel_err(val, ref.view_as(val))
            assert e <= tol, (case["name"], key, e)


def test_oracle_forward_matches_reference_cpu_op(op_cases):
    """Cross-check with the reference's own compiled CPU scan (sru/csrc/sru_cpu_impl.cpp:56-226)."""
    so = oracle_build.build_reference_cpu()
    if so is None or not os.path.exists(so):
        pytest.skip("reference CPU op not built on this machine")
    torch.ops.load_library(so)
    n = 0
    for case in op_cases:
        m = case["meta"]
        if case["mask_c"] is not None or m["custom"]:
            continue  # the CPU op has no dropout mask; its bi custom-V indexing differs (sru_cpu_impl.cpp:202)
        f = torch.float32
        dirs = m["dirs"]
        fn = torch.ops.sru_cpu.cpu_bi_forward if dirs == 2 else torch.ops.sru_cpu.cpu_forward
        mp = case["mask_pad"]
        h_ref, c_ref = fn(case["U"].to(f), case["x"].to(f), case["weight_c"].to(f), case["bias"].to(f),
                          case["c_init"].to(f), None if mp is None else mp.bool().contiguous(),
                          m["L"], m["B"], m["d"], m["k"], m["act"], m["has_skip"],
                          1.0 if m["scale"] is None else m["scale"], False)
        skip = 0 if not m["has_skip"] else (1 if m["k"] == 3 else 2)
        h, _, c_last = sru_oracle.forward(case["U"].to(f), case["x"].to(f), case["weight_c"].to(f),
                                          case["bias"].to(f), case["c_init"].to(f), None, mp,
                                          m["L"], m["B"], m["d"], dirs, m["k"], m["act"], skip, False,
                                          1.0 if m["scale"] is None else m["scale"])
        assert rel_err(h, h_ref) <= 1e-6, case["name"]
        assert rel_err(c_last, c_ref) <= 1e-6, case["name"]
        n += 1
    assert n >= 5


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-12), (torch.float32, 1e-5)])
def test_oracle_layer_norm_matches_reference(layer_norm_cases, dtype, tol):
    """The C restatement of layer normalisation against the reference's nn.LayerNorm (float64 vectors):
    output, input gradient, weight and bias gradients."""
    from oracle import sru_oracle
    for case in layer_norm_cases:
        x = case["x"].to(dtype)
        x2d = x.reshape(-1, case["n"])
        y, mean, rstd = sru_oracle.layer_norm_forward(x2d, case["weight"].to(dtype), case["bias"].to(dtype), case["eps"])
        dx, dg, db = sru_oracle.layer_norm_backward(case["dy"].to(dtype).reshape(-1, case["n"]), x2d, mean, rstd,
                                                    case["weight"].to(dtype))
        assert rel_err(y.view_as(case["y"]), case["y"]) <= tol, case["n"]
        assert rel_err(dx.view_as(case["dx"]), case["dx"]) <= tol, case["n"]
        assert rel_err(dg, case["dweight"]) <= tol, case["n"]
        assert rel_err(db, case["dbias"]) <= tol, case["n"]
