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


# ---------------------------------------------------------------------------------------------------------
# The model-level checker (oracle/ref_model.py: an independent restatement of the reference's layer stack)
# ---------------------------------------------------------------------------------------------------------
def test_oracle_model_matches_reference_model(model_cases):
    """OracleSRU with the reference's state dict against the reference's own sru.SRU on CPU: outputs, last
    states and every parameter gradient (LN before / after, residual, c0 split, low-rank chain, input
    projection, nn.RNN-style return, no-skip + tanh)."""
    from oracle.ref_model import from_state
    for case in model_cases:
        model = from_state(case["kwargs"], case["state"]).train()
        h, c = model(case["x"], case["c0"], mask_pad=case["mask_pad"])
        (h.sum() if case["loss"] == "sum" else (h ** 2).mean()).backward()
        assert (h - case["h"]).abs().max() <= 1e-5, case["name"]
        assert (c - case["c"]).abs().max() <= 1e-5, case["name"]
        grads = dict(model.named_parameters())
        assert set(case["grads"]) <= set(grads), case["name"]
        for n, ref in case["grads"].items():
            g = grads[n].grad
            # norm after the recurrence + loss h.sum(): gradients upstream of the norm are exactly zero and the
            # reference holds rounding noise there; judge those by absolute difference
            if float(ref.abs().max()) < 1e-6:
                assert float((g - ref).abs().max()) <= 1e-6, (case["name"], n)
            else:
                assert rel_err(g, ref) <= 2e-5, (case["name"], n)


def test_oracle_model_regression_artifact(regression_case):
    """The reference's own regression vector (sru 2.3.5, test/regression/test_regression.py:19-51), 1e-6."""
    from oracle.ref_model import from_state
    rc = regression_case
    model = from_state(rc["kwargs"], rc["state"]).eval()
    h, c = model(rc["x"])
    assert (h - rc["h"]).abs().max() <= 1e-6
    assert (c - rc["c"]).abs().max() <= 1e-6


def test_oracle_model_init_is_the_references(model_cases):
    """Same seed, same draws: OracleSRU's initialisation reproduces the reference's reset_parameters."""
    from oracle.ref_model import OracleSRU
    case = [c for c in model_cases if c["name"] == "config1"][0]
    kw = dict(case["kwargs"])
    torch.manual_seed(0)
    model = OracleSRU(kw.pop("input_size"), kw.pop("hidden_size"), **kw)
    sd = model.state_dict()
    assert list(sd.keys()) == list(case["state"].keys())
    for k, v in case["state"].items():
        assert torch.equal(sd[k], v), k


@pytest.mark.parametrize("kw", [
    dict(input_size=12, hidden_size=8, num_layers=3, bidirectional=True, layer_norm=True, rescale=True, dropout=0.2),
    dict(input_size=16, hidden_size=16, num_layers=2, projection_size=4, highway_bias=-3.0),
    dict(input_size=6, hidden_size=8, num_layers=2, proj_input_to_hidden_first=True, rnn_dropout=0.1,
         weight_c_init=0.5, normalize_after=True, layer_norm=True),
    dict(input_size=8, hidden_size=8, num_layers=2, v1=True, has_skip_term=False, use_tanh=True),
])
def test_oracle_model_and_shipped_model_initialise_alike(kw):
    """Two independent statements of the reference's recipe (the checker's and the shipped host code's) draw the
    same numbers from the same seed, for every branch of the recipe."""
    import warnings
    from oracle.ref_model import OracleSRU
    from sru_b200.modules import SRU
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        torch.manual_seed(5)
        a = SRU(**kw).state_dict()
        torch.manual_seed(5)
        k2 = dict(kw)
        b = OracleSRU(k2.pop("input_size"), k2.pop("hidden_size"), **k2).state_dict()
    assert list(a.keys()) == list(b.keys())
    for k in a:
        assert torch.equal(a[k], b[k]), k
