"""The boundary as a C++ application sees it (the reference's test/test.sh + test/test_ts_cpp.py +
sru/csrc/main_test_cpp.cpp): script a model, save it, run it from a C++ host that links the operator
binding, and compare the printed numbers (four decimals) with the Python run of the same module."""
import math
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _host():
    from sru_b200 import build
    path = build.TS_HOST
    if not os.path.exists(path):
        try:
            path = build.build_ts_host()
        except (OSError, subprocess.CalledProcessError) as e:      # no compiler on this machine
            pytest.skip("C++ host not built and cannot be built here: %s" % e)
    return path


def _lines(t):
    return "".join("{:.4f} ".format(v) for v in t.float().reshape(-1).tolist())


def _close(a, b, tol):
    fa, fb = [float(v) for v in a.split()], [float(v) for v in b.split()]
    return len(fa) == len(fb) and all(abs(x - y) <= tol for x, y in zip(fa, fb))


@pytest.mark.parametrize("kw,bf16", [
    (dict(), False),
    (dict(normalize_after=True, layer_norm=True), False),       # the two settings of the reference's test.sh
    (dict(layer_norm=True, bidirectional=True), False),
    (dict(input_size=64, hidden_size=64, bidirectional=True, layer_norm=True, projection_size=16), True),
])
def test_cpp_host_runs_scripted_model(tmp_path, kw, bf16):
    from sru_b200.modules import SRU
    host = _host()
    kw = dict(kw)
    n_in = kw.pop("input_size", 4)
    d = kw.pop("hidden_size", 4)
    torch.manual_seed(12)
    model = SRU(n_in, d, num_layers=2, **kw).eval()
    ts = torch.jit.script(model)
    path = str(tmp_path / "sru_ts.pt")
    ts.save(path)
    L, B = 5, 3
    x = torch.sin(torch.arange(L * B * n_in, dtype=torch.float32) * 0.37).view(L, B, n_in).to(DEV)
    model = model.to(DEV)
    if bf16:
        model, x = model.to(torch.bfloat16), x.to(torch.bfloat16)
    with torch.no_grad():
        h, c = model(x)                       # eager
        h2, c2 = torch.jit.script(model)(x)   # scripted, in Python
    expected = _lines(h) + "\n" + _lines(c) + "\n"
    res = subprocess.run([host, path] + (["bf16"] if bf16 else []), capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    got = res.stdout
    if not bf16:
        # fp32: identical text, as the reference's `diff cpp_out.txt py_out.txt` demands (a last-digit flip from
        # rounding at the fourth decimal is the only tolerated difference)
        assert got == expected or all(_close(g, e, 1.01e-4) for g, e in zip(got.splitlines(), expected.splitlines()))
        assert _lines(h2) == _lines(h)
    else:
        # bf16: eager keeps the gate bias in the GEMM epilogue, the scripted path adds it in the scan
        for g, e in zip(got.splitlines(), expected.splitlines()):
            assert _close(g, e, 2e-2 * max(1.0, float(h.float().abs().max())))
    assert len(got.splitlines()) == 2 and not any(math.isnan(float(v)) for v in got.split())
