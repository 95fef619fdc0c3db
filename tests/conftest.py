import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (sm_100a)")


# ---- parity report: every parity check may record the error it reached; the session prints a table and,
# when SRU_B200_PARITY_REPORT names a file, writes the records there as JSON ----
_PARITY = []


def record_parity(test, tensor, err, tol, note=""):
    _PARITY.append({"test": str(test), "tensor": str(tensor), "err": float(err), "tol": float(tol), "note": str(note)})


def check_parity(test, tensor, new, ref, tol, note=""):
    """rel_err(new, ref) <= tol, with the reached error recorded for the session's report."""
    e = rel_err(new, ref)
    record_parity(test, tensor, e, tol, note)
    assert e <= tol, (test, tensor, e, tol, note)
    return e


def pytest_terminal_summary(terminalreporter):
    if not _PARITY:
        return
    worst = {}
    for r in _PARITY:
        key = (r["test"], r["tensor"])
        if key not in worst or r["err"] / max(r["tol"], 1e-300) > worst[key]["err"] / max(worst[key]["tol"], 1e-300):
            worst[key] = r
    tr = terminalreporter
    tr.write_sep("-", "parity errors reached (max|new-ref| / max|ref|; worst case per test and tensor)")
    for (test, tensor), r in sorted(worst.items()):
        tr.write_line("%-58s %-14s err %.3e  tol %.1e  %s" % (test[:58], tensor[:14], r["err"], r["tol"], r["note"]))
    path = os.environ.get("SRU_B200_PARITY_REPORT")
    if path:
        import json
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump(sorted(worst.values(), key=lambda r: (r["test"], r["tensor"])), f, indent=1)


def rel_err(new, ref):
    """max|new - ref| / max(max|ref|, 1e-12), the error metric used for every parity check."""
    new = new.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert new.shape == ref.shape, (new.shape, ref.shape)
    if ref.numel() == 0:
        return 0.0
    return float((new - ref).abs().max() / max(float(ref.abs().max()), 1e-12))


@pytest.fixture(scope="session")
def op_cases():
    return torch.load(os.path.join(GOLDEN, "op_cases.pt"), weights_only=False)


@pytest.fixture(scope="session")
def model_cases():
    return torch.load(os.path.join(GOLDEN, "model_cases.pt"), weights_only=False)


@pytest.fixture(scope="session")
def regression_case():
    return torch.load(os.path.join(GOLDEN, "regression_2_3_5.pt"), weights_only=False)


@pytest.fixture(scope="session")
def layer_norm_cases():
    return torch.load(os.path.join(GOLDEN, "layer_norm_cases.pt"), weights_only=False)


@pytest.fixture
def host_on_cpu(monkeypatch):
    """Lets the shipped SRU / SRUCell host code run on CPU tensors, for this test only: the three device
    operations it calls are replaced by CPU ones (torch.mm, the oracle layer norm, the oracle scan).
    The package itself never routes anywhere but to its CUDA library."""
    from oracle import sru_oracle
    from sru_b200 import modules

    def real_of(t):
        return torch.float64 if t.dtype == torch.float64 else torch.float32

    def recurrence(U, x, V, bias, c0, act, d, bi, skip, scale=None, mask_c=None, mask_pad=None, amp16=False,
                   grad_link=None, bias_in_u=False):
        assert not bias_in_u
        dt = real_of(U)
        h, c = sru_oracle.elementwise_recurrence_oracle(
            U.to(dt), x.to(dt), V.to(dt), bias.to(dt), c0.to(dt), act, d, bi, skip,
            None if scale is None else scale.to(dt), None if mask_c is None else mask_c.to(dt), mask_pad)
        return [h, c]

    def project(x, w, col_bias=None, link=None):
        out = x.mm(w)
        return out if col_bias is None else out + col_bias.to(out.dtype)

    def layer_norm(t, w, b, eps=1e-5, out_dtype=None):
        return sru_oracle.layer_norm_oracle(t.to(real_of(t)), w, b, eps)

    monkeypatch.setattr(modules.ops, "elementwise_recurrence_gpu", recurrence)
    monkeypatch.setattr(modules, "project", project)
    monkeypatch.setattr(modules, "layer_norm", layer_norm)
    monkeypatch.setattr(modules, "grad_link_enabled", lambda: False)
    return modules
