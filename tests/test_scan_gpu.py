"""Parity of the CUDA scan kernels (called through the C ABI) with the CPU oracle.

Tolerances (relative to the largest magnitude of the reference tensor):
  fp64 1e-10, fp32 1e-5, bf16 / fp16 2e-2.
For 16-bit storage the oracle runs in fp32 on the same 16-bit-rounded inputs.
"""
import pytest
import torch

from conftest import record_parity, rel_err
from oracle import sru_oracle

pytestmark = pytest.mark.gpu

TOL = {torch.float64: 1e-10, torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def _ops():
    from sru_b200 import ops
    return ops


def _opts(**kw):
    from sru_b200 import _lib
    return _lib.options(**kw)


def run_both(case_inputs, dtype, c_dtype=None, need_grad=True, expect_kernel=None):
    """Runs oracle (CPU) and CUDA on the same (dtype-rounded) inputs; returns two dicts.
    expect_kernel: (forward, backward) kernel family the library must report for these calls."""
    ops = _ops()
    (U, x, wc, bias, c0, mc, mp, gh, gl, L, B, d, dirs, k, act, skip, custom, scale) = case_inputs
    d_ = d
    dev = torch.device("cuda:0")
    odt = torch.float64 if dtype == torch.float64 else torch.float32
    sm = odt
    Us, xs = U.to(dtype), x.to(dtype)
    wcs = wc.to(dtype) if custom else wc.to(sm)
    ghs = gh.to(dtype)
    # oracle on the rounded values
    oh, och, ocl = sru_oracle.forward(Us.to(odt), xs.to(odt), wcs.to(odt), bias.to(odt), c0.to(odt),
                                      None if mc is None else mc.to(odt), mp, L, B, d, dirs, k, act, skip,
                                      custom, scale)
    ref = dict(h=oh, c_last=ocl, c_hist=och)
    D = d * dirs
    cu = lambda t: None if t is None else t.to(dev).contiguous()
    pad = None if mp is None else mp.bool().to(dev).contiguous()
    h, c_hist, c_last = ops.scan_forward(cu(Us), cu(xs) if skip == 1 else None, cu(wcs), cu(bias.to(sm)),
                                         cu(c0.to(sm)), cu(None if mc is None else mc.to(sm)), pad,
                                         L, B, d, dirs, k, act, skip, int(custom), scale, True, c_dtype)
    out = dict(h=h, c_last=c_last, c_hist=c_hist)
    from sru_b200 import _lib as _l
    allowed = lambda e: (e,) if isinstance(e, str) else tuple(e)
    if expect_kernel is not None:
        assert _l.last_scan_kernel() in allowed(expect_kernel[0]), (_l.last_scan_kernel(), expect_kernel)
    if need_grad:
        # the oracle's backward consumes ITS c history; the kernel consumes its own
        ogu, ogx, ogwc, ogb, ogi = sru_oracle.backward(
            Us.to(odt), xs.to(odt), wcs.to(odt), bias.to(odt), c0.to(odt),
            None if mc is None else mc.to(odt), mp, och, ghs.to(odt), gl.to(odt),
            L, B, d, dirs, k, act, skip, custom, scale)
        ref.update(grad_u=ogu, grad_x=ogx, grad_wc=ogwc, grad_bias=ogb, grad_init=ogi)
        gu, gx, gwc, gb, gi = ops.scan_backward(
            cu(Us), cu(xs) if skip == 1 else None, cu(wcs), cu(bias.to(sm)), cu(c0.to(sm)),
            cu(None if mc is None else mc.to(sm)), pad, c_hist, cu(ghs), cu(gl.to(sm)),
            L, B, d, dirs, k, act, skip, int(custom), scale)
        out.update(grad_u=gu, grad_x=gx, grad_wc=gwc, grad_bias=gb, grad_init=gi)
        if expect_kernel is not None:
            assert _l.last_scan_kernel() in allowed(expect_kernel[1]), (_l.last_scan_kernel(), expect_kernel)
    torch.cuda.synchronize()
    from sru_b200 import _lib
    _lib.check_device_error()
    if dtype == torch.float32:
        # The recurrence amplifies rounding differences over long sequences (its Jacobian is not
        # contractive for arbitrary weight_c), so two correct fp32 implementations drift apart.
        # Judge both against the fp64 oracle on the same inputs: `ref` becomes the fp64 result and
        # ref["_fp32_drift"] holds how far the fp32 ORACLE itself is from it, per tensor.
        d = torch.float64
        f = lambda t: None if t is None else t.to(d)
        oh, och, ocl = sru_oracle.forward(f(Us), f(xs), f(wcs), f(bias.float()), f(c0.float()),
                                          f(None if mc is None else mc.float()), mp, L, B, d_, dirs, k, act,
                                          skip, custom, float(torch.tensor(scale, dtype=torch.float32)))
        ref64 = dict(h=oh, c_last=ocl, c_hist=och)
        if need_grad:
            r = sru_oracle.backward(f(Us), f(xs), f(wcs), f(bias.float()), f(c0.float()),
                                    f(None if mc is None else mc.float()), mp, och, f(ghs), f(gl.float()),
                                    L, B, d_, dirs, k, act, skip, custom,
                                    float(torch.tensor(scale, dtype=torch.float32)))
            ref64.update(grad_u=r[0], grad_x=r[1], grad_wc=r[2], grad_bias=r[3], grad_init=r[4])
        drift = {key: (0.0 if v is None else rel_err(ref[key].reshape(v.shape), v)) for key, v in ref64.items()}
        # Conditioning: how far the EXACT (fp64) results move when U is perturbed by half an fp32 ulp
        # (relative 6e-8, random signs).  No fp32 computation can be expected to come closer than that;
        # on random data the adjoint recurrence amplifies such perturbations up to a few 1e-5 at L ~ 70.
        sign = torch.sign(torch.randn(Us.shape, generator=torch.Generator().manual_seed(7))).to(d)
        Up = f(Us) * (1 + 6e-8 * sign)
        ph, pch, pcl = sru_oracle.forward(Up, f(xs), f(wcs), f(bias.float()), f(c0.float()),
                                          f(None if mc is None else mc.float()), mp, L, B, d_, dirs, k, act,
                                          skip, custom, float(torch.tensor(scale, dtype=torch.float32)))
        pert = dict(h=ph, c_last=pcl, c_hist=pch)
        if need_grad:
            r = sru_oracle.backward(Up, f(xs), f(wcs), f(bias.float()), f(c0.float()),
                                    f(None if mc is None else mc.float()), mp, pch, f(ghs), f(gl.float()),
                                    L, B, d_, dirs, k, act, skip, custom,
                                    float(torch.tensor(scale, dtype=torch.float32)))
            pert.update(grad_u=r[0], grad_x=r[1], grad_wc=r[2], grad_bias=r[3], grad_init=r[4])
        for key, v in ref64.items():
            if v is not None:
                drift[key] = max(drift[key], rel_err(pert[key].reshape(v.shape), v))
        ref = ref64
        ref["_fp32_drift"] = drift
    return out, ref


FP32_CAP = 6e-5      # no conditioning argument widens the fp32 bar beyond this (largest error reached: 5.2e-5)


def compare(out, ref, tol, tag):
    """Every tensor of `out` against `ref` at `tol`; the error reached goes into the session's parity report.

    fp32 only: `ref` is then the fp64 oracle and carries, per tensor, how far the exact result moves under a
    half-ulp perturbation of U and how far the fp32 CPU oracle itself lands from it ("drift").  A well-conditioned
    case (4 x drift <= 1e-5) is held to the strict 1e-5; an ill-conditioned one to 4 x drift, never beyond FP32_CAP
    (of 587 fp32 checks in a run, 8 exceed 1e-5, all on 71-step sequences with random padding).
    """
    drift = ref.get("_fp32_drift", {})
    for key, r in ref.items():
        if key == "_fp32_drift":
            continue
        if r is None:
            assert out[key] is None, (tag, key)
            continue
        e = rel_err(out[key].reshape(r.shape), r)
        eff, note = tol, ""
        if key in drift:
            eff = min(max(tol, 4.0 * drift[key]), FP32_CAP)
            note = "fp32; drift %.1e" % drift[key]
        record_parity(tag, key, e, eff, note)
        assert e <= eff, (tag, key, e, eff, drift.get(key))


def golden_inputs(case, ):
    m = case["meta"]
    skip = 0 if not m["has_skip"] else (1 if m["k"] == 3 else 2)
    return (case["U"], case["x"], case["weight_c"], case["bias"], case["c_init"], case["mask_c"],
            case["mask_pad"], case["grad_h"], case["grad_last"], m["L"], m["B"], m["d"], m["dirs"],
            m["k"], m["act"], skip, bool(m["custom"]), 1.0 if m["scale"] is None else m["scale"])


def random_inputs(L, B, d, dirs, k, skip=None, pad=None, maskc=True, c0=True, scale=1.0, seed=0,
                  custom=False, act=0):
    g = torch.Generator().manual_seed(seed)
    D = d * dirs
    if skip is None:
        skip = 1 if k == 3 else 2
    U = torch.randn(L, B, D * k, generator=g)
    x = torch.randn(L, B, D, generator=g)
    wc = torch.randn(L, B, D * 2, generator=g) if custom else torch.randn(2 * D, generator=g)
    bias = torch.randn(2 * D, generator=g)
    c0t = torch.randn(B, D, generator=g) if c0 else torch.zeros(B, D)
    mc = ((torch.rand(B, D, generator=g) > 0.2).float() / 0.8) if maskc else None
    mp = None
    if pad == "tail":
        lens = torch.randint(max(1, L // 2), L + 1, (B,), generator=g)
        mp = torch.arange(L).view(L, 1) >= lens.view(1, B)
    elif pad == "random":
        mp = torch.rand(L, B, generator=g) > 0.7
    gh = torch.randn(L, B, D, generator=g)
    gl = torch.randn(B, D, generator=g)
    return (U, x, wc, bias, c0t, mc, mp, gh, gl, L, B, d, dirs, k, act, skip, custom, scale)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("force_generic", [0, 1])
def test_golden_cases(op_cases, dtype, force_generic):
    """Golden vectors of the reference's elementwise_recurrence_naive, outputs and all gradients."""
    with _opts(force_generic=force_generic):
        for case in op_cases:
            inp = golden_inputs(case)
            out, _ = run_both(inp, dtype, expect_kernel=("generic", "generic") if force_generic else None)
            tol = TOL[dtype]
            gold = dict(h=case["h"], c_last=case["c_last"], grad_u=case["grad_U"], grad_x=case["grad_x"],
                        grad_wc=case["grad_weight_c"], grad_bias=case["grad_bias"],
                        grad_init=case["grad_c_init"])
            compare({k: out[k] for k in gold}, gold, tol, case["name"])


SHAPES = [
    # L,  B,  d,  dirs, k, pad
    (9,   3,  8,   1, 3, None),
    (13,  5,  16,  2, 3, "tail"),
    (7,   4,  32,  2, 4, "random"),
    (33,  7,  64,  1, 3, "tail"),
    (20,  32, 128, 1, 3, None),       # first benchmark configuration's layer shape
    (17,  9,  304, 1, 3, "tail"),     # hidden size of the reference's AMP test (not a power of two)
    (41,  6,  128, 2, 4, "tail"),
    (5,   33, 256, 2, 3, "random"),
    (64,  2,  512, 1, 3, None),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", SHAPES)
def test_pipelined_vs_oracle(shape, dtype):
    L, B, d, dirs, k, pad = shape
    inp = random_inputs(L, B, d, dirs, k, pad=pad, scale=1.3, seed=L * 131 + B)
    for c_dtype in ([None] if dtype == torch.float32 else [torch.float32, dtype]):
        out, ref = run_both(inp, dtype, c_dtype, expect_kernel=(("pipelined", "split"), "pipelined"))
        compare(out, ref, TOL[dtype], (shape, dtype, c_dtype))


@pytest.mark.parametrize("v", [1, 2, 4])
@pytest.mark.parametrize("threads", [32, 64, 128])
@pytest.mark.parametrize("stages", [2, 5])
def test_pipelined_tilings(v, threads, stages):
    """Every columns-per-thread / CTA size / ring depth the dispatcher can pick gives the same answer."""
    for dtype in (torch.float32, torch.bfloat16):
        s = 4 if dtype == torch.float32 else 2
        if v * s > 16:
            continue
        for (L, B, d, dirs, k, pad) in [(11, 5, 64, 2, 3, "tail"), (6, 3, 128, 1, 4, "random")]:
            inp = random_inputs(L, B, d, dirs, k, pad=pad, seed=v * 7 + threads)
            with _opts(fwd_v=v, bwd_v=v, scan_threads=threads, scan_stages=stages, fwd_split=0):
                out, ref = run_both(inp, dtype, expect_kernel=("pipelined", "pipelined"))
            compare(out, ref, TOL[dtype], (v, threads, stages, dtype, L, B, d, dirs, k))


@pytest.mark.parametrize("ss", [4, 8, 32])
@pytest.mark.parametrize("v,threads", [(1, 64), (2, 64), (4, 64)])
def test_pad_flags_across_stages(v, threads, ss):
    """mask_pad reaches the kernels through the producer warp, one pipeline stage ahead: sequences that
    span many stages and several trips round a two-stage ring, several batch rows per tile (the last tile
    short of rows), both directions, random and tail padding."""
    for pad in ("random", "tail"):
        inp = random_inputs(71, 7, 64, 2, 3, pad=pad, seed=ss + v)
        with _opts(fwd_v=v, bwd_v=v, scan_threads=threads, scan_stages=2, scan_ss=ss, fwd_split=0):
            out, ref = run_both(inp, torch.bfloat16, expect_kernel=("pipelined", "pipelined"))
        compare(out, ref, TOL[torch.bfloat16], (v, threads, ss, pad))
        with _opts(fwd_v=min(v, 2), bwd_v=v, scan_threads=threads, scan_stages=3, scan_ss=ss, fwd_split=0):
            out, ref = run_both(inp, torch.float32, expect_kernel=("pipelined", "pipelined"))
        compare(out, ref, TOL[torch.float32], (v, threads, ss, pad, "fp32"))


def test_edge_cases_empty_single_and_fully_padded():
    """Zero-length and zero-batch calls return empty outputs and pass the initial state through; one step and one
    sequence work; a sequence that is padding from the first step keeps c_init, gives h = 0 and passes grad_last
    through to grad_init."""
    ops = _ops()
    dev = "cuda:0"
    d, dirs, k = 64, 2, 3
    D = d * dirs
    g = torch.Generator().manual_seed(77)
    wc, bias = torch.randn(2 * D, generator=g).to(dev), torch.randn(2 * D, generator=g).to(dev)
    for (L, B) in ((0, 3), (4, 0)):
        U = torch.empty(L, B, D * k, device=dev, dtype=torch.bfloat16)
        x = torch.empty(L, B, D, device=dev, dtype=torch.bfloat16)
        c0 = torch.randn(B, D, generator=g).to(dev)
        h, ch, cl = ops.scan_forward(U, x, wc, bias, c0, None, None, L, B, d, dirs, k, 0, 1, 0, 1.0)
        assert h.shape == (L, B, D) and ch.shape == (L, B, D) and torch.equal(cl, c0)
        gl = torch.randn(B, D, generator=g).to(dev)
        gu, gx, gwc, gb, gi = ops.scan_backward(U, x, wc, bias, c0, None, None, ch, torch.empty_like(x), gl,
                                                L, B, d, dirs, k, 0, 1, 0, 1.0)
        assert gu.shape == U.shape and float(gwc.abs().sum()) == 0.0 and torch.equal(gi, gl)
    for (L, B) in ((1, 1), (1, 5), (6, 1)):
        inp = random_inputs(L, B, d, dirs, k, pad=None, seed=L * 10 + B)
        out, ref = run_both(inp, torch.bfloat16)
        compare(out, ref, TOL[torch.bfloat16], ("single", L, B))
    # sequence 1 of 3 is padding everywhere
    L, B = 12, 3
    inp = list(random_inputs(L, B, d, dirs, k, pad="tail", seed=5))
    mp = inp[6].clone()
    mp[:, 1] = True
    inp[6] = mp
    out, ref = run_both(tuple(inp), torch.float32)
    compare(out, ref, TOL[torch.float32], "fully padded")
    c0, gl = inp[4], inp[8]
    assert float(out["h"][:, 1].abs().max()) == 0.0
    assert torch.equal(out["c_last"][1].cpu(), c0[1]) and torch.equal(out["grad_init"][1].cpu(), gl[1])
    assert float(out["grad_u"].view(L, B, -1)[:, 1].abs().max()) == 0.0


def test_options_no_skip_no_bias_no_c0():
    ops = _ops()
    inp = list(random_inputs(10, 4, 64, 2, 3, skip=0, pad="tail", maskc=False, c0=False, seed=5))
    out, ref = run_both(tuple(inp), torch.float32)
    compare(out, ref, 1e-5, "noskip")
    # bias == NULL means "already folded into U": equal to a zero bias
    (U, x, wc, bias, c0, mc, mp, gh, gl, L, B, d, dirs, k, act, skip, custom, scale) = inp
    dev = "cuda:0"
    h0, _, cl0 = ops.scan_forward(U.to(dev), None, wc.to(dev), torch.zeros_like(bias).to(dev), None, None,
                                  mp.to(dev), L, B, d, dirs, k, act, skip, 0, 1.0)
    h1, _, cl1 = ops.scan_forward(U.to(dev), None, wc.to(dev), None, None, None,
                                  mp.to(dev), L, B, d, dirs, k, act, skip, 0, 1.0)
    assert torch.equal(h0, h1) and torch.equal(cl0, cl1)


def test_inference_without_history_matches():
    ops = _ops()
    inp = random_inputs(37, 6, 128, 1, 3, pad=None, seed=11)
    (U, x, wc, bias, c0, mc, mp, gh, gl, L, B, d, dirs, k, act, skip, custom, scale) = inp
    dev = "cuda:0"
    a = ops.scan_forward(U.to(dev), x.to(dev), wc.to(dev), bias.to(dev), c0.to(dev), None, None,
                         L, B, d, dirs, k, act, skip, 0, 1.0, True)
    b = ops.scan_forward(U.to(dev), x.to(dev), wc.to(dev), bias.to(dev), c0.to(dev), None, None,
                         L, B, d, dirs, k, act, skip, 0, 1.0, False)
    assert b[1] is None and torch.equal(a[0], b[0]) and torch.equal(a[2], b[2])
    # last state equals the last row of the history
    assert torch.equal(a[1][-1], a[2])


def test_bad_arguments_are_reported():
    from sru_b200 import _lib
    L = _lib.lib()
    rc = L.sru_b200_scan_forward(None, None, None, None, None, None, None, None, None, None,
                                 4, 2, 8, 3, 3, 0, 1, 0, 1.0, 0, 0, None)
    assert rc == -1 and b"dirs" in L.sru_b200_last_error()
    rc = L.sru_b200_scan_forward(None, None, None, None, None, None, None, None, None, None,
                                 4, 2, 8, 1, 4, 0, 1, 0, 1.0, 0, 0, None)
    assert rc == -1 and b"skip_type 1" in L.sru_b200_last_error()
    rc = L.sru_b200_scan_backward(*([None] * 15), 4, 2, 8, 1, 3, 0, 1, 0, 1.0, 0, 0, None, 0, None)
    assert rc == -1


def test_autograd_function_matches_oracle_autograd():
    """elementwise_recurrence_gpu (public operator) against the oracle through torch.autograd."""
    ops = _ops()
    for bi, k in ((False, 3), (True, 4), (True, 3)):
        dirs = 2 if bi else 1
        L, B, d = 12, 5, 32
        inp = random_inputs(L, B, d, dirs, k, pad="tail", scale=1.4, seed=77 + k)
        (U, x, wc, bias, c0, mc, mp, gh, gl, *_rest) = inp
        leaves = [t.clone().requires_grad_(True) for t in (U, x, wc, bias, c0)]
        sx = torch.tensor([1.4])
        h, cl = sru_oracle.elementwise_recurrence_oracle(*leaves, 0, d, bi, True, sx, mc, mp)
        ((h * gh).sum() + (cl * gl).sum()).backward()
        dev = "cuda:0"
        gleaves = [t.detach().clone().to(dev).requires_grad_(True) for t in (U, x, wc, bias, c0)]
        h2, cl2 = ops.elementwise_recurrence_gpu(*gleaves, 0, d, bi, True, sx.to(dev), mc.to(dev), mp.to(dev))
        ((h2 * gh.to(dev)).sum() + (cl2 * gl.to(dev)).sum()).backward()
        assert rel_err(h2, h) <= 1e-5 and rel_err(cl2, cl) <= 1e-5
        for a, b, name in zip(gleaves, leaves, "U x wc bias c0".split()):
            if k == 4 and name == "x":
                assert a.grad is None or float(a.grad.abs().max()) == 0.0
                continue
            assert rel_err(a.grad, b.grad) <= 1e-5, (bi, k, name)


def test_config2_first_layer_scan_at_size():
    """The k = 4 first layer of benchmark configuration 2 at its full size (L=256, B=64, bidirectional 512 per
    direction, bf16 storage, tail padding, unscaled N(0,1) inputs): every output and gradient against the oracle."""
    inp = random_inputs(256, 64, 512, 2, 4, pad="tail", scale=1.0, seed=2024)
    out, ref = run_both(inp, torch.bfloat16, expect_kernel=(("pipelined", "split"), "pipelined"))
    compare(out, ref, TOL[torch.bfloat16], "config2 layer0 scan k=4")


def _guarded(nbytes, dtype):
    """A device tensor of nbytes / itemsize elements of `dtype` inside a buffer with 256-byte guard bands of 0xA5."""
    raw = torch.full((nbytes + 512,), 0xA5, dtype=torch.uint8, device="cuda:0")
    return raw, raw[256:256 + nbytes].view(dtype)


def _bands_intact(raw, nbytes):
    return bool((raw[:256] == 0xA5).all()) and bool((raw[256 + nbytes:] == 0xA5).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [
    # L,  B, d, dirs, k     ragged everywhere: B not a multiple of the rows per tile, L not of the stage length
    (13,  5, 8,  1, 3),    # hidden = one 16-byte granule of bf16 (two of fp32)
    (37,  7, 64, 2, 3),
    (9,   3, 16, 2, 4),
    (131, 33, 128, 1, 3),
])
def test_no_write_outside_the_outputs(shape, dtype):
    """Every output and the workspace sit between guard bands; after forward and backward through the C ABI the
    bands are untouched and the results equal those of the ordinary call path (stand-in for a memory checker)."""
    from sru_b200 import _lib
    ops = _ops()
    L, B, d, dirs, k = shape
    D = d * dirs
    inp = random_inputs(L, B, d, dirs, k, pad="tail", scale=1.2, seed=L + B)
    (U, x, wc, bias, c0, mc, mp, gh, gl, *_r) = inp
    dev = "cuda:0"
    es = 2 if dtype == torch.bfloat16 else 4
    Us, xs, ghs = U.to(dtype).to(dev), x.to(dtype).to(dev), gh.to(dtype).to(dev)
    wcd, bd, c0d, mcd, gld = wc.to(dev), bias.to(dev), c0.to(dev), mc.to(dev), gl.to(dev)
    pad = mp.to(dev).contiguous()
    skip = 1 if k == 3 else 2
    lib = _lib.lib()
    code = _lib.DTYPE_CODE[dtype]
    st = _lib.current_stream_ptr()
    n = L * B * D
    raw_h, h = _guarded(n * es, dtype)
    raw_c, ch = _guarded(n * 4, torch.float32)
    raw_l, cl = _guarded(B * D * 4, torch.float32)
    rc = lib.sru_b200_scan_forward(h.data_ptr(), ch.data_ptr(), cl.data_ptr(), Us.data_ptr(),
                                   xs.data_ptr() if skip == 1 else None, wcd.data_ptr(), bd.data_ptr(), c0d.data_ptr(),
                                   mcd.data_ptr(), pad.data_ptr(), L, B, d, dirs, k, 0, skip, 0, 1.2, code, 0, st)
    assert rc == 0, lib.sru_b200_last_error()
    fwd_kernel = _lib.last_scan_kernel()
    raw_gu, gu = _guarded(n * k * es, dtype)
    raw_gx, gx = _guarded(n * es, dtype)
    raw_gw, gwc = _guarded(2 * D * 4, torch.float32)
    raw_gb, gb = _guarded(2 * D * 4, torch.float32)
    raw_gi, gi = _guarded(B * D * 4, torch.float32)
    wbytes = int(lib.sru_b200_scan_backward_workspace_bytes(L, B, d, dirs, k, code))
    raw_ws, ws = _guarded(wbytes, torch.uint8)
    rc = lib.sru_b200_scan_backward(gu.data_ptr(), gx.data_ptr() if skip == 1 else None, gwc.data_ptr(), gb.data_ptr(),
                                    gi.data_ptr(), Us.data_ptr(), xs.data_ptr() if skip == 1 else None, wcd.data_ptr(),
                                    bd.data_ptr(), c0d.data_ptr(), mcd.data_ptr(), pad.data_ptr(), ch.data_ptr(),
                                    ghs.data_ptr(), gld.data_ptr(), L, B, d, dirs, k, 0, skip, 0, 1.2, code, 0,
                                    ws.data_ptr(), wbytes, st)
    assert rc == 0, lib.sru_b200_last_error()
    torch.cuda.synchronize()
    _lib.check_device_error()
    assert fwd_kernel in ("pipelined", "split") and _lib.last_scan_kernel() == "pipelined"
    for name, raw, nb in (("h", raw_h, n * es), ("c_hist", raw_c, n * 4), ("c_last", raw_l, B * D * 4),
                          ("grad_u", raw_gu, n * k * es), ("grad_x", raw_gx, n * es), ("grad_wc", raw_gw, 2 * D * 4),
                          ("grad_bias", raw_gb, 2 * D * 4), ("grad_init", raw_gi, B * D * 4), ("workspace", raw_ws, wbytes)):
        assert _bands_intact(raw, nb), (name, shape, dtype)
    # same results as the ordinary path (fresh allocations)
    h2, ch2, cl2 = ops.scan_forward(Us, xs if skip == 1 else None, wcd, bd, c0d, mcd, pad, L, B, d, dirs, k, 0, skip,
                                    0, 1.2, True, torch.float32)
    r = ops.scan_backward(Us, xs if skip == 1 else None, wcd, bd, c0d, mcd, pad, ch2, ghs, gld, L, B, d, dirs, k, 0,
                          skip, 0, 1.2)
    assert torch.equal(h.view(L, B, D), h2) and torch.equal(ch.view(L, B, D), ch2) and torch.equal(cl.view(B, D), cl2)
    assert torch.equal(gu.view(L, B, D * k), r[0]) and torch.equal(gi.view(B, D), r[4])
    assert torch.equal(gwc, r[2]) and torch.equal(gb, r[3])
    if skip == 1:
        assert torch.equal(gx.view(L, B, D), r[1])


def test_options_interface():
    from sru_b200 import _lib
    assert _lib.get_option("fwd_v") == -1
    with _lib.options(fwd_v=2):
        assert _lib.get_option("fwd_v") == 2
    assert _lib.get_option("fwd_v") == -1
    with pytest.raises(_lib.SruB200Error):
        _lib.set_option("no_such_option", 1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("v", [1, 2])
@pytest.mark.parametrize("shape", [
    # L,  B,  d,  dirs, k, pad,    threads, stages, ss
    (37,  6, 128, 1, 3, None,     128, None, None),
    (71,  7, 64,  2, 3, "tail",   64,  2,    4),
    (19,  3, 32,  2, 4, "random", 32,  3,    8),
    (130, 2, 256, 1, 3, "random", 128, 2,    32),
    (5,   9, 16,  2, 4, "tail",   64,  None, None),
])
def test_split_role_forward(shape, v, dtype):
    """The forward kernel with the state chain and the output work on separate warps: against the oracle, and bit
    for bit against the one-role pipelined kernel (same operations per column), with and without a state history."""
    from sru_b200 import _lib
    ops = _ops()
    L, B, d, dirs, k, pad, threads, stages, ss = shape
    inp = random_inputs(L, B, d, dirs, k, pad=pad, scale=1.3, seed=L * 17 + B + v)
    with _opts(fwd_split=1, fwd_v=v, scan_threads=threads, scan_stages=stages, scan_ss=ss):
        out, ref = run_both(inp, dtype, expect_kernel=("split", "pipelined"))
        compare(out, ref, TOL[dtype], ("split", shape, v, dtype))
    (U, x, wc, bias, c0, mc, mp, gh, gl, *_r) = inp
    dev = "cuda:0"
    skip = 1 if k == 3 else 2
    args = (U.to(dtype).to(dev), x.to(dtype).to(dev) if skip == 1 else None, wc.to(dev), bias.to(dev), c0.to(dev),
            mc.to(dev), None if mp is None else mp.to(dev), L, B, d, dirs, k, 0, skip, 0, 1.3)
    for hist in (True, False):
        with _opts(fwd_split=1, fwd_v=v, scan_threads=threads, scan_stages=stages, scan_ss=ss):
            a = ops.scan_forward(*args, hist)
            assert _lib.last_scan_kernel() == "split"
        with _opts(fwd_split=0, fwd_v=v, scan_threads=threads, scan_stages=stages, scan_ss=ss):
            b = ops.scan_forward(*args, hist)
            assert _lib.last_scan_kernel() == "pipelined"
        assert torch.equal(a[0], b[0]) and torch.equal(a[2], b[2])
        if hist:
            assert torch.equal(a[1], b[1])
    torch.cuda.synchronize()
    _lib.check_device_error()


def test_nvtx_ranges():
    """NVTX ranges around the library's launches (for profiler filters) change nothing else."""
    from sru_b200 import _lib
    inp = random_inputs(33, 5, 64, 2, 3, pad="tail", scale=1.0, seed=91)
    out0, ref = run_both(inp, torch.bfloat16)
    _lib.set_nvtx_ranges(True)
    try:
        out1, _ = run_both(inp, torch.bfloat16)
    finally:
        _lib.set_nvtx_ranges(False)
    for k in out0:
        assert torch.equal(out0[k], out1[k]), k
