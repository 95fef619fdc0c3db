"""The allocation-free backward entry point (sru_b200_scan_backward_noalloc) against the regular one.

Some hosts of this library may not allocate GPU memory around a call (fixed memory plans,
sandboxes without an allocator), so this entry point keeps its scratch inside the library.
The test drives it through the C ABI with ctypes, twice in a row with different problems, and
checks every output against sru_b200_scan_backward given a caller-allocated workspace: the
same kernels run, so the results must be bit-identical.  It also checks that a problem beyond
the built-in scratch is refused with a clear message.  Collected last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

_vp, _i64, _int = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int


def _entry_points():
    from sru_b200 import _lib
    L = _lib.lib()
    fn = L.sru_b200_scan_backward_noalloc
    fn.restype = _int
    fn.argtypes = [_vp] * 15 + [_i64, _i64, _i64, _int, _int, _int, _int, _int, ctypes.c_double, _int, _int, _vp]
    L.sru_b200_scan_backward_noalloc_max_bytes.restype = ctypes.c_size_t
    return L, fn


def _problem(L, B, d, dirs, k, dtype, seed):
    from sru_b200 import ops
    g = torch.Generator().manual_seed(seed)
    D = d * dirs
    U = torch.randn(L, B, D * k, generator=g).to(dtype).to(DEV)
    x = torch.randn(L, B, D, generator=g).to(dtype).to(DEV) if k == 3 else None
    wc = torch.randn(2 * D, generator=g).to(DEV)
    bias = torch.randn(2 * D, generator=g).to(DEV)
    c0 = torch.randn(B, D, generator=g).to(DEV)
    mc = ((torch.rand(B, D, generator=g) > 0.2).float() / 0.8).to(DEV)
    lens = torch.randint(max(1, L // 2), L + 1, (B,), generator=g)
    pad = (torch.arange(L).view(L, 1) >= lens.view(1, B)).to(DEV)
    gh = torch.randn(L, B, D, generator=g).to(dtype).to(DEV)
    gl = torch.randn(B, D, generator=g).to(DEV)
    skip = 1 if k == 3 else 2
    h, c_hist, c_last = ops.scan_forward(U, x, wc, bias, c0, mc, pad, L, B, d, dirs, k, 0, skip, 0, 1.25)
    return dict(U=U, x=x, wc=wc, bias=bias, c0=c0, mc=mc, pad=pad, gh=gh, gl=gl, c_hist=c_hist,
                L=L, B=B, d=d, dirs=dirs, k=k, skip=skip, dtype=dtype)


def _run(p, noalloc):
    from sru_b200 import _lib
    L, fn = _entry_points()
    D = p["d"] * p["dirs"]
    dt = p["dtype"]
    gu = torch.empty_like(p["U"])
    gx = torch.empty(p["L"], p["B"], D, dtype=dt, device=DEV) if p["skip"] == 1 else None
    gwc = torch.empty(2 * D, device=DEV)
    gb = torch.empty(2 * D, device=DEV)
    gi = torch.empty(p["B"], D, device=DEV)
    ptr = _lib.ptr
    code, ccode = _lib.DTYPE_CODE[dt], _lib.DTYPE_CODE[p["c_hist"].dtype]
    head = (ptr(gu), ptr(gx), ptr(gwc), ptr(gb), ptr(gi), ptr(p["U"]), ptr(p["x"]), ptr(p["wc"]), ptr(p["bias"]),
            ptr(p["c0"]), ptr(p["mc"]), ptr(p["pad"]), ptr(p["c_hist"]), ptr(p["gh"]), ptr(p["gl"]),
            p["L"], p["B"], p["d"], p["dirs"], p["k"], 0, p["skip"], 0, 1.25, code, ccode)
    stream = _lib.current_stream_ptr()
    if noalloc:
        rc = fn(*head, stream)
    else:
        nbytes = L.sru_b200_scan_backward_workspace_bytes(p["L"], p["B"], p["d"], p["dirs"], p["k"], code)
        ws = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=DEV)
        rc = L.sru_b200_scan_backward(*head, ptr(ws), ws.numel(), stream)
    assert rc == 0, L.sru_b200_last_error()
    torch.cuda.synchronize()
    return [t for t in (gu, gx, gwc, gb, gi) if t is not None]


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    from sru_b200 import _lib
    problems = [
        _problem(37, 6, 128, 2, 3, torch.bfloat16, seed=1),   # pipelined kernels
        _problem(9, 5, 7, 1, 3, torch.float32, seed=2),       # generic kernels (odd hidden size)
        _problem(21, 3, 64, 1, 4, torch.float32, seed=3),
    ]
    for p in problems:
        expected = _run(p, noalloc=False)
        first = _run(p, noalloc=True)
        second = _run(p, noalloc=True)      # the shared scratch still holds the previous call's partials
        for e, a, b in zip(expected, first, second):
            assert torch.equal(e, a) and torch.equal(e, b)
    _lib.check_device_error()


def test_noalloc_refuses_problems_beyond_its_scratch():
    L, fn = _entry_points()
    limit = L.sru_b200_scan_backward_noalloc_max_bytes()
    assert limit == 8 << 20
    # batch * dirs * hidden = 1024 * 2 * 512 = 1048576 > 524288: refused before anything is touched
    rc = fn(*([None] * 15), 4, 1024, 512, 2, 3, 0, 1, 0, 1.0, 0, 0, None)
    assert rc == -3
    msg = L.sru_b200_last_error().decode()
    assert "scratch" in msg and str(limit) in msg
    # one column beyond the limit is refused, again before any pointer is looked at
    rc = fn(*([None] * 15), 4, 524289, 1, 1, 3, 0, 1, 0, 1.0, 0, 0, None)
    assert rc == -3


def test_noalloc_accepts_a_problem_exactly_at_its_limit():
    """batch * dirs * hidden = 256 * 2 * 1024 = 524288 columns need exactly the 8 MiB the library holds."""
    from sru_b200 import _lib
    L, fn = _entry_points()
    p = _problem(4, 256, 1024, 2, 3, torch.bfloat16, seed=4)
    code = _lib.DTYPE_CODE[torch.bfloat16]
    assert L.sru_b200_scan_backward_workspace_bytes(4, 256, 1024, 2, 3, code) == L.sru_b200_scan_backward_noalloc_max_bytes()
    expected = _run(p, noalloc=False)
    got = _run(p, noalloc=True)
    for e, a in zip(expected, got):
        assert torch.equal(e, a)
    _lib.check_device_error()
