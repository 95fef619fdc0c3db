"""Model-level parity on the GPU: SRU / SRUCell of this package against the reference's golden
vectors and against the CPU oracle model, eager and TorchScript, fp32 and autocast."""
import pytest
import torch

from conftest import rel_err
from oracle.cpu_model import to_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sru():
    from sru_b200.modules import SRU
    return SRU


def _loss(h, kind):
    return h.sum() if kind == "sum" else (h ** 2).mean()


def test_golden_model_cases(model_cases):
    """Forward, last states and every parameter gradient of the reference's sru.SRU (CPU, fp32);
    the absolute bound 1e-4 is the reference's own CPU-vs-GPU test bound (test/sru/test_sru.py:129)."""
    SRU = _sru()
    for case in model_cases:
        model = SRU(**case["kwargs"])
        model.load_state_dict(case["state"], strict=True)
        model = model.to(DEV).train()
        mp = None if case["mask_pad"] is None else case["mask_pad"].to(DEV)
        c0 = None if case["c0"] is None else case["c0"].to(DEV)
        h, c = model(case["x"].to(DEV), c0, mask_pad=mp)
        _loss(h, case["loss"]).backward()
        assert h.dtype == torch.float32 and c.dtype == torch.float32
        assert (h.cpu() - case["h"]).abs().max() <= 1e-4, case["name"]
        assert (c.cpu() - case["c"]).abs().max() <= 1e-4, case["name"]
        assert rel_err(h, case["h"]) <= 1e-5 and rel_err(c, case["c"]) <= 1e-5, case["name"]
        for n, p in model.named_parameters():
            if n in case["grads"]:
                assert (p.grad.cpu() - case["grads"][n]).abs().max() <= 1e-4, (case["name"], n)
                if float(case["grads"][n].abs().max()) > 1e-3:  # post-LN + sum loss gives ~0 gradients
                    assert rel_err(p.grad, case["grads"][n]) <= 2e-5, (case["name"], n)


def test_regression_artifact(regression_case):
    """Golden vector of sru 2.3.5 (test/regression/test_regression.py:19-51), bound 1e-6."""
    rc = regression_case
    model = _sru()(**rc["kwargs"]).eval()
    model.load_state_dict(rc["state"], strict=True)
    model = model.to(DEV)
    with torch.no_grad():
        h, c = model(rc["x"].to(DEV))
    assert (h.cpu() - rc["h"]).abs().max() <= 1e-6
    assert (c.cpu() - rc["c"]).abs().max() <= 1e-6


@pytest.mark.parametrize("bidirectional", [False, True])
@pytest.mark.parametrize("layer_norm", [False, True])
def test_batch_independence(bidirectional, layer_norm):
    """Final state of a padded batch equals each sequence run alone (test/sru/test_sru.py:6-78)."""
    torch.manual_seed(3)
    model = _sru()(7, 4, num_layers=5, bidirectional=bidirectional, layer_norm=layer_norm).to(DEV).eval()
    lens = [4, 2, 3]
    L = max(lens)
    x = torch.randn(L, len(lens), 7, device=DEV)
    mp = torch.tensor([[t >= n for n in lens] for t in range(L)], device=DEV)
    for grad in (False, True):
        with torch.set_grad_enabled(grad):
            _, c = model(x, mask_pad=mp)
            for i, n in enumerate(lens):
                _, ci = model(x[:n, i:i + 1].contiguous())
                assert (c[:, i] - ci[:, 0]).abs().max() <= 1e-4


@pytest.mark.parametrize("bidirectional", [False, True])
@pytest.mark.parametrize("proj", [0, 4])
@pytest.mark.parametrize("layer_norm", [False, True])
def test_torchscript_equals_eager(bidirectional, proj, layer_norm):
    """eager(grad) == eager(no_grad) == scripted (test/sru/test_torchscript.py:6-53), bound 1e-4."""
    torch.manual_seed(5)
    model = _sru()(32, 32, num_layers=2, bidirectional=bidirectional, rescale=True, projection_size=proj,
                   layer_norm=layer_norm).to(DEV).eval()
    x = torch.randn(16, 8, 32, device=DEV)
    h1, c1 = model(x)
    with torch.no_grad():
        h2, c2 = model(x)
        ts = torch.jit.script(model)
        h3, c3 = ts(x)
    for a, b in ((h1, h2), (c1, c2), (h1, h3), (c1, c3)):
        assert (a - b).abs().max() <= 1e-4


@pytest.mark.parametrize("amp_dtype", [torch.bfloat16, torch.float16])
def test_autocast_native_and_reference_modes(amp_dtype):
    """Autocast training step: both amp modes return what the reference returns in dtype
    (fp32 h and c, fp32 parameter gradients), and values within 2e-2 of the fp32 CPU oracle
    that is fed the same 16-bit-rounded weights and input."""
    import sru_b200
    torch.manual_seed(11)
    SRU = _sru()
    kw = dict(input_size=64, hidden_size=64, num_layers=3, bidirectional=True, layer_norm=True, rescale=True,
              dropout=0.0)
    model = SRU(**kw).to(DEV).train()
    L, B = 24, 6
    x = torch.randn(L, B, 64, device=DEV)
    lens = torch.randint(12, L + 1, (B,))
    mp = (torch.arange(L).view(L, 1) >= lens.view(1, B)).to(DEV)
    cpu = to_oracle(model).train()
    h_ref, c_ref = cpu(x.cpu(), mask_pad=mp.cpu())
    h_ref.sum().backward()
    ref_grads = {n: p.grad for n, p in cpu.named_parameters()}
    for mode in ("native", "reference"):
        sru_b200.set_amp_mode(mode)
        try:
            model.zero_grad()
            with torch.autocast("cuda", dtype=amp_dtype):
                h, c = model(x, mask_pad=mp)
                loss = h.float().sum()
            loss.backward()
        finally:
            sru_b200.set_amp_mode("native")
        assert h.dtype == torch.float32 and c.dtype == torch.float32, mode
        assert rel_err(h, h_ref) <= 2e-2, (mode, rel_err(h, h_ref))
        assert rel_err(c, c_ref) <= 2e-2, mode
        for n, p in model.named_parameters():
            assert p.grad.dtype == torch.float32
            assert rel_err(p.grad, ref_grads[n]) <= 2e-2, (mode, n, rel_err(p.grad, ref_grads[n]))


@pytest.mark.parametrize("amp_dtype", [torch.bfloat16, torch.float16])
def test_grad_link_equals_autograd_sum(amp_dtype, monkeypatch):
    """Layers 1.. of a k = 3 stack use their input as GEMM operand and as highway term.  With the gradient
    link the dgrad GEMM accumulates onto the scan's grad_x; without it autograd adds the two.  Same gradients
    (one 16-bit rounding apart), and both within 2e-2 of the fp32 CPU oracle."""
    import sru_b200
    from sru_b200 import projection
    torch.manual_seed(5)
    SRU = _sru()
    model = SRU(input_size=64, hidden_size=64, num_layers=3, bidirectional=True, dropout=0.0).to(DEV).train()
    L, B = 19, 8
    x0 = torch.randn(L, B, 64, device=DEV)
    lens = torch.randint(9, L + 1, (B,))
    mp = (torch.arange(L).view(L, 1) >= lens.view(1, B)).to(DEV)
    cpu = to_oracle(model).train()
    xr = x0.cpu().requires_grad_(True)
    h_ref, _ = cpu(xr, mask_pad=mp.cpu())
    (h_ref * h_ref).sum().backward()
    ref = {n: p.grad for n, p in cpu.named_parameters()}
    ref["x"] = xr.grad

    accumulating = []
    real_gemm = projection.gemm

    def spy(*a, **kw):
        accumulating.append(bool(kw.get("accumulate", False)))
        return real_gemm(*a, **kw)
    monkeypatch.setattr(projection, "gemm", spy)

    got = {}
    for on in (True, False):
        projection.set_grad_link_enabled(on)
        accumulating.clear()
        try:
            model.zero_grad()
            x = x0.clone().requires_grad_(True)
            with torch.autocast("cuda", dtype=amp_dtype):
                h, _ = model(x, mask_pad=mp)
                loss = (h.float() ** 2).sum()
            loss.backward()
        finally:
            projection.set_grad_link_enabled(True)
        # two of the three layers (128 -> 128, k = 3) qualify; the first (64 -> 128, k = 4) does not
        assert sum(accumulating) == (2 if on else 0), (on, accumulating)
        got[on] = {n: p.grad.clone() for n, p in model.named_parameters()}
        got[on]["x"] = x.grad.clone()
    for n in got[True]:
        assert rel_err(got[True][n], got[False][n]) <= 1e-2, (n, rel_err(got[True][n], got[False][n]))
        assert rel_err(got[True][n], ref[n]) <= 2e-2, (n, rel_err(got[True][n], ref[n]))


def test_dropout_mask_is_an_input():
    """With the same RNG state the training-mode dropout mask equals the oracle model's."""
    torch.manual_seed(2)
    model = _sru()(16, 16, num_layers=3, dropout=0.3).to(DEV).train()
    x = torch.randn(9, 4, 16, device=DEV)
    masks = []
    orig = type(model.rnn_lst[0]).get_dropout_mask_

    def record(self, size, p):
        m = orig(self, size, p)
        masks.append(m.cpu())
        return m

    cpu = to_oracle(model).train()
    for cell in model.rnn_lst:
        cell.get_dropout_mask_ = record.__get__(cell)
    h, c = model(x)
    it = iter(masks)
    cpu.mask_source = lambda li, like, size, p: next(it)
    h_ref, c_ref = cpu(x.cpu())
    assert len(masks) == 2  # no dropout after the last layer
    assert rel_err(h, h_ref) <= 1e-5 and rel_err(c, c_ref) <= 1e-5


def test_sru_cuda_ops_backward_match_python_path():
    """The registered sru_cuda::* backward operators against the ctypes path (same kernels)."""
    from sru_b200 import _lib, ops
    _lib.load_torch_ops()
    g = torch.Generator().manual_seed(9)
    L, B, d = 10, 3, 16
    for bi in (False, True):
        D = d * (2 if bi else 1)
        U = torch.randn(L, B, D * 3, generator=g).to(DEV)
        x = torch.randn(L, B, D, generator=g).to(DEV)
        wc, bias = torch.randn(2 * D, generator=g).to(DEV), torch.randn(2 * D, generator=g).to(DEV)
        c0 = torch.randn(B, D, generator=g).to(DEV)
        gh, gl = torch.randn(L, B, D, generator=g).to(DEV), torch.randn(B, D, generator=g).to(DEV)
        fwd = torch.ops.sru_cuda.sru_bi_forward_simple if bi else torch.ops.sru_cuda.sru_forward_simple
        bwd = torch.ops.sru_cuda.sru_bi_backward_simple if bi else torch.ops.sru_cuda.sru_backward_simple
        h, c = fwd(U, x, wc, bias, c0, None, None, L, B, d)
        gu, gx, gwc, gb, gi = bwd(U, x, wc, bias, c0, None, None, c, gh, gl, L, B, d)
        h2, c2, cl2 = ops.scan_forward(U, x, wc, bias, c0, None, None, L, B, d, 2 if bi else 1, 3, 0, 1, 0, 1.0)
        r = ops.scan_backward(U, x, wc, bias, c0, None, None, c2, gh, gl, L, B, d, 2 if bi else 1, 3, 0, 1, 0, 1.0)
        assert torch.equal(h, h2) and torch.equal(c, c2)
        assert torch.equal(gu, r[0]) and torch.equal(gx, r[1]) and torch.equal(gi, r[4])
        assert torch.equal(gwc.sum(1).view(-1), r[2]) and torch.equal(gb.sum(1).view(-1), r[3])


def test_sru_cuda_general_backward_ops():
    """sru_cuda::sru_backward / sru_bi_backward (the general operators: k = 4, tanh, custom per-step V) against the
    ctypes path with the same arguments."""
    from sru_b200 import _lib, ops
    _lib.load_torch_ops()
    g = torch.Generator().manual_seed(19)
    L, B, d = 9, 4, 16
    for bi, k, act, custom in ((False, 4, 0, False), (True, 4, 1, False), (False, 3, 1, True), (True, 4, 0, True)):
        dirs = 2 if bi else 1
        D = d * dirs
        skip = 1 if k == 3 else 2
        U = torch.randn(L, B, D * k, generator=g).to(DEV)
        x = torch.randn(L, B, D, generator=g).to(DEV)
        wc = (torch.randn(L, B, D * 2, generator=g) if custom else torch.randn(2 * D, generator=g)).to(DEV)
        bias, c0 = torch.randn(2 * D, generator=g).to(DEV), torch.randn(B, D, generator=g).to(DEV)
        mc = ((torch.rand(B, D, generator=g) > 0.2).float() / 0.8).to(DEV)
        pad = (torch.rand(L, B, generator=g) > 0.7).to(DEV)
        gh, gl = torch.randn(L, B, D, generator=g).to(DEV), torch.randn(B, D, generator=g).to(DEV)
        fwd = torch.ops.sru_cuda.sru_bi_forward if bi else torch.ops.sru_cuda.sru_forward
        bwd = torch.ops.sru_cuda.sru_bi_backward if bi else torch.ops.sru_cuda.sru_backward
        xin = x if skip == 1 else None
        h, c = fwd(U, xin, wc, bias, c0, mc, pad, L, B, d, k, act, skip, int(custom))
        gu, gx, gwc, gb, gi = bwd(U, xin, wc, bias, c0, mc, pad, c, gh, gl, L, B, d, k, act, skip, int(custom))
        h2, c2, _ = ops.scan_forward(U, xin, wc, bias, c0, mc, pad, L, B, d, dirs, k, act, skip, int(custom), 1.0)
        r = ops.scan_backward(U, xin, wc, bias, c0, mc, pad, c2, gh, gl, L, B, d, dirs, k, act, skip, int(custom), 1.0)
        assert _lib.last_scan_kernel() == ("generic" if (custom or act) else "pipelined")
        assert torch.equal(h, h2) and torch.equal(c, c2)
        assert torch.equal(gu, r[0]) and torch.equal(gi, r[4])
        if skip == 1:
            assert torch.equal(gx, r[1])
        if custom:
            assert torch.equal(gwc, r[2])
        else:
            assert torch.equal(gwc.sum(1).view(-1), r[2])
        assert torch.equal(gb.sum(1).view(-1), r[3])


@pytest.mark.parametrize("amp_dtype", [torch.bfloat16, torch.float16])
def test_bias_in_gemm_epilogue_equals_bias_in_scan(amp_dtype):
    """Gate bias added by the projection's epilogue (default for 16-bit projections) against the bias added inside the
    scan: same outputs and gradients to 16-bit rounding, both within 2e-2 of the oracle; highway bias -3, k = 4 first
    layer and k = 3 layers, low-rank chain."""
    from sru_b200 import projection
    for kw in (dict(input_size=64, hidden_size=128, num_layers=3, bidirectional=True, highway_bias=-3.0),
               dict(input_size=128, hidden_size=128, num_layers=2, projection_size=32, highway_bias=-1.5, rescale=True)):
        torch.manual_seed(21)
        model = _sru()(**kw).to(DEV).train()
        with torch.no_grad():
            for cell in model.rnn_lst:
                cell.bias.add_(torch.randn_like(cell.bias) * 0.5)
        L, B = 33, 8
        x = torch.randn(L, B, kw["input_size"], generator=torch.Generator().manual_seed(3)).to(DEV)
        cpu = to_oracle(model, round_to=amp_dtype).train()
        h_ref, _ = cpu(x.cpu().to(amp_dtype).float())
        (h_ref ** 2).mean().backward()
        ref = {n: p.grad for n, p in cpu.named_parameters()}
        got = {}
        for fold in (True, False):
            projection.set_bias_fold_enabled(fold)
            try:
                model.zero_grad()
                with torch.autocast("cuda", dtype=amp_dtype):
                    h, _ = model(x)
                    loss = (h.float() ** 2).mean()
                loss.backward()
            finally:
                projection.set_bias_fold_enabled(True)
            got[fold] = dict({n: p.grad.clone() for n, p in model.named_parameters()}, h=h.detach())
            assert rel_err(h, h_ref) <= 2e-2
        for n in got[True]:
            assert rel_err(got[True][n], got[False][n]) <= 1e-2, (n, rel_err(got[True][n], got[False][n]))
            if n != "h":
                assert rel_err(got[True][n], ref[n]) <= 2e-2, (n, rel_err(got[True][n], ref[n]))


def test_scale_x_changes_take_effect():
    """The scalar the kernels take for scale_x is remembered between calls; every way the module itself changes the
    buffer (reset_parameters, load_state_dict, versioned in-place ops) and forget_scale after a raw .data write
    must reach the next forward."""
    from sru_b200 import ops
    torch.manual_seed(6)
    model = _sru()(16, 16, num_layers=1, rescale=True).to(DEV).eval()
    cell = model.rnn_lst[0]
    x = torch.randn(5, 2, 16, device=DEV)
    cpu = to_oracle(model).eval()

    def agree():
        with torch.no_grad():
            h, _ = model(x)
            cpu.rnn_lst[0].scale_x.copy_(cell.scale_x.cpu())
            oh, _ = cpu(x.cpu())
        return rel_err(h, oh) <= 1e-5

    assert agree()
    with torch.no_grad():
        cell.scale_x.fill_(2.5)                     # versioned in-place write
    assert agree()
    cell.scale_x.data[0] = 0.75                     # the reference's own idiom: invisible to the version counter
    ops.forget_scale(cell.scale_x)
    assert agree()
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    sd["rnn_lst.0.scale_x"] = torch.tensor([1.9])
    model.load_state_dict(sd)
    assert agree()
    cell.reset_parameters()
    cpu = to_oracle(model).eval()
    assert agree()


@pytest.mark.parametrize("kwargs,L,B,in_size,use_mask,use_c0", [
    (dict(hidden_size=64, num_layers=3), 24, 8, 64, False, False),                         # k = 3 everywhere
    (dict(hidden_size=64, num_layers=3, bidirectional=True), 31, 8, 40, True, True),       # k = 4 first layer, padding
    (dict(hidden_size=128, num_layers=2, highway_bias=-2.0, rescale=True), 16, 4, 128, True, False),
    (dict(hidden_size=32, num_layers=2, has_skip_term=False), 8, 8, 32, False, True),
    (dict(hidden_size=64, num_layers=3, bidirectional=True, layer_norm=True), 20, 8, 128, True, False),   # pre-norm
    (dict(hidden_size=64, num_layers=2, layer_norm=True, normalize_after=True), 12, 4, 48, False, True),  # post-norm
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_native_layer_loop_matches_python_loop(kwargs, L, B, in_size, use_mask, use_c0, dtype):
    """Inference through ``sru_b200::stack_forward`` (the layer loop as one native call) gives the bits of the
    Python loop over the layers: same kernels, same arguments.  Under autocast on fp32 input and on 16-bit input
    with 16-bit weights, with and without layer norms; stacks it does not serve (a factorised projection) keep
    the Python loop."""
    from sru_b200 import _lib, modules
    SRU = _sru()
    torch.manual_seed(L + B)
    model = SRU(in_size, **kwargs).to(DEV).eval()
    D = model.output_size
    x = torch.randn(L, B, in_size, device=DEV)
    mask = None
    if use_mask:
        lens = torch.randint(L // 2, L + 1, (B,))
        mask = (torch.arange(L).view(L, 1) >= lens.view(1, B)).to(DEV)
    c0 = torch.randn(model.num_layers, B, D, device=DEV) * 0.3 if use_c0 else None

    def run(native, autocast):
        modules.set_native_stack_enabled(native)
        try:
            n0 = _lib.launch_count
            with torch.no_grad():
                if autocast:
                    with torch.autocast("cuda", dtype=dtype):
                        h, c = model(x, c0, mask_pad=mask)
                else:
                    m16 = SRU(in_size, **kwargs).to(DEV).eval()
                    m16.load_state_dict(model.state_dict())
                    m16 = m16.to(dtype)
                    h, c = m16(x.to(dtype), None if c0 is None else c0.to(dtype), mask_pad=mask)
            return h, c, _lib.launch_count - n0
        finally:
            modules.set_native_stack_enabled(True)
    for autocast in (True, False):
        h1, c1, n1 = run(True, autocast)
        h0, c0_, n0 = run(False, autocast)
        torch.cuda.synchronize()
        _lib.check_device_error()
        assert h1.dtype == h0.dtype and c1.dtype == c0_.dtype and h1.shape == h0.shape and c1.shape == c0_.shape
        assert torch.equal(h1, h0) and torch.equal(c1, c0_)
        norms = model.num_layers if kwargs.get("layer_norm") else 0
        widen = 1 if autocast else 0                       # float32 input under autocast: h comes back as float32
        assert n0 == 3 * model.num_layers + norms + widen  # Python loop: bias layout, product, scan (+ norm) per layer
        assert n1 in (n0, n0 - model.num_layers)           # native loop: the bias layout is kept between calls
    # the copies kept between calls follow in-place updates of the parameters
    with torch.no_grad():
        model.rnn_lst[0].weight.mul_(0.5)
        model.rnn_lst[-1].bias.add_(0.25)
    ha, ca, _ = run(True, True)
    hb, cb, _ = run(False, True)
    assert torch.equal(ha, hb) and torch.equal(ca, cb) and not torch.equal(ha, h1)
    # not served: falls back to the Python loop and still works
    pj = SRU(in_size, projection_size=16, **kwargs).to(DEV).eval()
    n0 = _lib.launch_count
    with torch.no_grad(), torch.autocast("cuda", dtype=dtype):
        h, c = pj(x, mask_pad=mask)
    assert torch.isfinite(h.float()).all() and _lib.launch_count - n0 > 3 * pj.num_layers


@pytest.mark.parametrize("n", [8, 13, 4096 + 3, 1 << 20])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_widening_cast_matches_the_framework(n, dtype):
    """The conversion kernel behind the module's float32 output: the bits of ``Tensor.float()`` going up and of
    ``Tensor.to(dtype)`` (round to nearest even, infinities, NaN-ness) coming back as the gradient."""
    from sru_b200 import _lib, ops
    g = torch.Generator().manual_seed(n)
    t = (torch.randn(n, generator=g) * 50).to(dtype).to(DEV)
    t[:3] = torch.tensor([float("inf"), -0.0, 65504.0 if dtype == torch.float16 else 3.3e38], dtype=dtype)
    leaf = t.clone().requires_grad_(True)
    up = ops.widen_to_float32(leaf)
    assert up.dtype == torch.float32 and torch.equal(up, t.float())
    grad = torch.randn(n, generator=g).to(DEV) * 1e3
    grad[:2] = torch.tensor([float("nan"), 1e39], device=DEV)
    up.backward(grad)
    want = grad.to(dtype)
    assert leaf.grad.dtype == dtype
    assert torch.equal(torch.isnan(leaf.grad), torch.isnan(want))
    assert torch.equal(torch.nan_to_num(leaf.grad.float()), torch.nan_to_num(want.float()))
    # what the kernel does not take goes to the framework
    view = t.view(-1)[1:] if n > 8 else t[::2]
    assert torch.equal(ops.widen_to_float32(view), view.float())
    torch.cuda.synchronize()
    _lib.check_device_error()


def test_streaming_chunks_equal_one_pass():
    """``StreamingSRU``: a unidirectional stack fed in chunks (state handed on) gives the bits of one pass over the
    whole sequence, for chunks whose projection runs on the same GEMM; bidirectional stacks are refused."""
    from sru_b200.streaming import StreamingSRU
    SRU = _sru()
    torch.manual_seed(5)
    model = SRU(64, 64, num_layers=3, layer_norm=True).to(DEV).eval()
    L, B = 96, 8
    x = torch.randn(L, B, 64, device=DEV)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        h_all, c_all = model(x)
        stream = StreamingSRU(model)
        parts = [stream.step(x[a:b]) for a, b in ((0, 16), (16, 17), (17, 64), (64, 96))]
    assert torch.equal(torch.cat(parts, 0), h_all) and torch.equal(stream.state, c_all)
    stream.reset()
    assert stream.state is None
    with pytest.raises(ValueError):
        StreamingSRU(SRU(64, 64, bidirectional=True))


def test_device_prefetcher_yields_the_batches_in_order():
    """``DevicePrefetcher``: batch i + 1 is copied on a side stream while batch i is in use; the consumer sees every
    batch, in order, with the host values, and None entries pass through."""
    from sru_b200.data import DevicePrefetcher
    g = torch.Generator().manual_seed(1)
    host = [(torch.randn(64, 8, 32, generator=g).pin_memory(), None if i % 2 else (torch.rand(64, 8, generator=g) > 0.5).pin_memory())
            for i in range(5)]
    seen = 0
    acc = torch.zeros((), device=DEV)
    for i, (x, m) in enumerate(DevicePrefetcher(iter(host), DEV)):
        assert x.is_cuda and torch.equal(x.cpu(), host[i][0])
        assert (m is None) == (host[i][1] is None) and (m is None or torch.equal(m.cpu(), host[i][1]))
        acc += (x * 2).sum()          # work on the consumer's stream while the next copy runs
        seen += 1
    assert seen == 5
    assert abs(float(acc) - 2 * sum(float(h[0].sum()) for h in host)) < 1e-1
    assert list(DevicePrefetcher(iter([]), DEV)) == []
    with pytest.raises(ValueError):
        DevicePrefetcher(iter(host), "cpu")
