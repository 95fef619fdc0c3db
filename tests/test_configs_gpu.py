"""The benchmark configurations at their full sizes, through the public module API (``SRU.forward`` +
``backward``), against the independent CPU oracle model (oracle/ref_model.py).

Weights come from the reference's default initialisation (same seed, same draws), inputs are the
seeded synthetic inputs of the benchmark, UNSCALED.  Since a full-size CPU run would take minutes to
hours, each configuration is checked the way batch-independent work allows:

* outputs, final states and the input gradient of three sampled batch rows of the full-size GPU run
  against the oracle run on just those rows (rows never interact; the loss is normalised by the global
  element count on both sides, and the GPU's dropout masks are replayed into the oracle);
* every parameter gradient on a reduced-batch re-run (batch 4, full length, full width) of the same
  model against the oracle on the same reduced batch.

Bar: 2e-2 relative to the largest magnitude of the reference tensor (16-bit storage), error recorded
per tensor.  The oracle computes in float32 with the projection weights (and the first layer's input
where it enters a GEMM directly) rounded to the autocast type.  fp16 runs use a static loss scale, as
the reference's AMP test does with its GradScaler (test/test_amp.py:60-75).
"""
import pytest
import torch

from conftest import check_parity, rel_err
from oracle.ref_model import to_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL16 = 2e-2


def _sru():
    from sru_b200.modules import SRU
    return SRU


def _inputs(cfg_id, L, B, n_in, x_std, lens):
    g = torch.Generator().manual_seed(1000 + cfg_id)
    x = torch.randn(L, B, n_in, generator=g) * x_std
    mask = None
    if lens is not None:
        n = torch.randint(lens[0], lens[1] + 1, (B,), generator=g)
        mask = torch.arange(L).view(L, 1) >= n.view(1, B)
    return x, mask


def _record_masks(model):
    """Wraps every layer's dropout-mask draw so that the masks of the next forward are kept (on the CPU)."""
    store = {}
    for li, cell in enumerate(model.rnn_lst):
        orig = type(cell).get_dropout_mask_

        def draw(size, p, _cell=cell, _li=li, _orig=orig):
            m = _orig(_cell, size, p)
            store.setdefault(_li, []).append(m.detach().float().cpu())
            return m
        cell.get_dropout_mask_ = draw
    return store


def _loss(h, kind, n_elements):
    hf = h.float()
    return hf.sum() if kind == "sum" else (hf * hf).sum() / float(n_elements)


def _gpu_step(model, x, mask, c0, amp, loss_kind, n_elements, loss_scale):
    store = _record_masks(model)
    model.zero_grad(set_to_none=True)
    xd = x.to(DEV).requires_grad_(True)
    md = None if mask is None else mask.to(DEV)
    with torch.autocast("cuda", dtype=amp):
        h, c = model(xd, c0, mask_pad=md)
    (_loss(h, loss_kind, n_elements) * loss_scale).backward()
    torch.cuda.synchronize()
    from sru_b200 import _lib
    _lib.check_device_error()
    for cell in model.rnn_lst:
        del cell.get_dropout_mask_
    masks = {li: v[0] for li, v in store.items()}
    grads = {n: (p.grad.detach().float() / loss_scale).cpu() for n, p in model.named_parameters() if p.grad is not None}
    return h.detach(), c.detach(), (xd.grad.detach() / loss_scale), masks, grads


def _oracle_step(model, x_rows, mask_rows, c0_rows, masks_rows, amp, loss_kind, n_elements, first_layer_has_norm):
    ref = to_oracle(model, round_to=amp).train()
    ref.mask_source = lambda li, like, size, p: masks_rows[li]
    xr = x_rows if first_layer_has_norm else x_rows.to(amp).float()     # what the first GEMM sees
    xr = xr.clone().requires_grad_(True)
    h, c = ref(xr, c0_rows, mask_pad=mask_rows)
    _loss(h, loss_kind, n_elements).backward()
    return h.detach(), c.detach(), xr.grad, {n: p.grad for n, p in ref.named_parameters() if p.grad is not None}


def _check_config(name, cfg_id, kwargs, L, B, amp, x_std=1.0, lens=None, use_c0=False, loss_kind="sum",
                  loss_scale=1.0, out_dtype=torch.float32, c_dtype=torch.float32, small_B=4):
    SRU = _sru()
    torch.manual_seed(0)
    model = SRU(**kwargs).to(DEV).train()
    dirs = 2 if kwargs.get("bidirectional") else 1
    D = kwargs["hidden_size"] * dirs
    nl = kwargs.get("num_layers", 2)
    has_norm = bool(kwargs.get("layer_norm")) and not kwargs.get("normalize_after")
    x, mask = _inputs(cfg_id, L, B, kwargs["input_size"], x_std, lens)
    n_el = L * B * D

    # ---- full size on the GPU; three batch rows against the oracle ----
    c0 = torch.zeros(nl, B, D, device=DEV) if use_c0 else None
    h, c, gx, masks, _ = _gpu_step(model, x, mask, c0, amp, loss_kind, n_el, loss_scale)
    assert h.dtype == out_dtype and c.dtype == c_dtype, (h.dtype, c.dtype)
    assert h.shape == (L, B, D) and c.shape == (nl, B, D)
    rows = [0, B // 2 - 1, B - 1]
    masks_rows = {li: m[rows] for li, m in masks.items()}
    oh, oc, ogx, _ = _oracle_step(model, x[:, rows].contiguous(), None if mask is None else mask[:, rows].contiguous(),
                                  torch.zeros(nl, len(rows), D) if use_c0 else None, masks_rows, amp, loss_kind,
                                  n_el, has_norm)
    check_parity(name, "h", h[:, rows], oh, TOL16, "3 rows of the full-size run")
    check_parity(name, "c_last", c[:, rows], oc, TOL16, "3 rows of the full-size run")
    check_parity(name, "grad_x", gx[:, rows], ogx, TOL16, "3 rows of the full-size run")
    if mask is not None:
        assert float((h * mask.to(DEV).unsqueeze(-1)).abs().max()) == 0.0      # padded positions give h = 0
    del h, c, gx

    # ---- reduced batch, same model: every parameter gradient ----
    xs = x[:, :small_B].contiguous()
    ms = None if mask is None else mask[:, :small_B].contiguous()
    n_small = L * small_B * D
    c0s = torch.zeros(nl, small_B, D, device=DEV) if use_c0 else None
    h, c, gx, masks, grads = _gpu_step(model, xs, ms, c0s, amp, loss_kind, n_small, loss_scale)
    oh, oc, ogx, ograds = _oracle_step(model, xs, ms, torch.zeros(nl, small_B, D) if use_c0 else None, masks, amp,
                                       loss_kind, n_small, has_norm)
    check_parity(name, "h(batch %d)" % small_B, h, oh, TOL16)
    assert set(grads) == set(ograds), (sorted(grads), sorted(ograds))
    for n in sorted(grads):
        assert grads[n].dtype == torch.float32
        check_parity(name, "grad " + n.replace("rnn_lst.", "L"), grads[n], ograds[n], TOL16, "batch %d" % small_B)


def test_config2_full_size():
    """Configuration 2: 4-layer bidirectional SRU 512 -> 512 per direction, pre-layer-norm, rescale (scale_x = sqrt 3),
    bf16 autocast, L=256, B=64, tail padding from lengths in [128, 256]; first layer k = 4 (512 -> 1024)."""
    _check_config("config2", 2, dict(input_size=512, hidden_size=512, num_layers=4, bidirectional=True,
                                     layer_norm=True, rescale=True),
                  L=256, B=64, amp=torch.bfloat16, lens=(128, 256), loss_kind="sum")


@pytest.mark.parametrize("fp16_recurrence", [False, True])
def test_config3_full_size(fp16_recurrence):
    """Configuration 3: 6-layer SRU 2048 with the low-rank chain 2048 -> 512 -> 6144, highway bias -3, fp16 autocast,
    x ~ N(0, 0.5), c0 = zeros, loss = mean of squares; both settings of amp_recurrence_fp16 (with it the caller
    gets h and the final states in half precision, as from the reference)."""
    half = torch.float16 if fp16_recurrence else torch.float32
    _check_config("config3/fp16_recurrence=%d" % fp16_recurrence, 3,
                  dict(input_size=2048, hidden_size=2048, num_layers=6, projection_size=512, highway_bias=-3.0,
                       amp_recurrence_fp16=fp16_recurrence),
                  L=512, B=32, amp=torch.float16, x_std=0.5, use_c0=True, loss_kind="meansq", loss_scale=65536.0,
                  out_dtype=half, c_dtype=half)


def test_config5_first_layers_full_size():
    """Configuration 5 at full length, batch and width, first three of its twelve layers (memory): layer 0 is the
    120 -> 2048 k = 4 layer (GEMM 256 000 x 8192 x 120, weight gradient 120 x 8192 over K = 256 000, cut into K
    slabs), layers 1-2 the 2048 -> 2048 k = 3 layers; dropout 0.1 after layers 0 and 1, tail padding, bf16."""
    _check_config("config5[3 layers]", 5, dict(input_size=120, hidden_size=1024, num_layers=3, bidirectional=True,
                                               dropout=0.1),
                  L=1000, B=256, amp=torch.bfloat16, lens=(600, 1000), loss_kind="meansq")


def test_config4_full_size_through_the_module():
    """Configuration 4 through SRU.forward: 1-layer SRU 1024, bf16 parameters and input, no grad, L=8192, B=16;
    h and the final state of two batch rows.  Then the same input in 8 chunks of 1024 steps, each chunk starting
    from the previous chunk's final state: bit-identical to the one-shot run (the long-sequence streaming pattern
    of language_model/train_enwik8.py:183-193)."""
    SRU = _sru()
    torch.manual_seed(0)
    model = SRU(1024, 1024, num_layers=1).to(torch.bfloat16).to(DEV).eval()
    L, B = 8192, 16
    x, _ = _inputs(4, L, B, 1024, 1.0, None)
    xd = x.to(torch.bfloat16).to(DEV)
    with torch.no_grad():
        h, c = model(xd)
    assert h.dtype == torch.bfloat16 and h.shape == (L, B, 1024) and c.shape == (1, B, 1024)
    rows = [2, 15]
    ref = to_oracle(model, round_to=torch.bfloat16).eval()
    with torch.no_grad():
        oh, oc = ref(xd[:, rows].float().cpu())
    check_parity("config4", "h", h[:, rows], oh, TOL16, "2 rows")
    check_parity("config4", "c_last", c[:, rows], oc, TOL16, "2 rows")
    with torch.no_grad():
        state = None
        parts = []
        for t0 in range(0, L, 1024):
            hp, state = model(xd[t0:t0 + 1024], state)
            parts.append(hp)
    assert torch.equal(torch.cat(parts), h) and torch.equal(state, c)


def test_chunked_training_step_equals_one_shot():
    """Two chunks chained through the final state WITH its gradient (grad_init of the second chunk flows into
    grad_last of the first) give the gradients of the one-shot step: uni-directional 3-layer stack, bf16."""
    SRU = _sru()
    torch.manual_seed(4)
    model = SRU(256, 256, num_layers=3, highway_bias=-1.0).to(DEV).train()
    L, B = 96, 8
    x = torch.randn(L, B, 256, generator=torch.Generator().manual_seed(5)).to(DEV)

    def grads(chunks):
        model.zero_grad(set_to_none=True)
        state, total = None, 0.0
        with torch.autocast("cuda", dtype=torch.bfloat16):
            for t0 in range(0, L, L // chunks):
                h, state = model(x[t0:t0 + L // chunks], state)
                total = total + (h.float() ** 2).sum()
        (total / float(L * B * 256)).backward()
        return {n: p.grad.clone() for n, p in model.named_parameters()}

    one, two = grads(1), grads(2)
    for n in one:
        check_parity("chunked_training", "grad " + n.replace("rnn_lst.", "L"), two[n], one[n], TOL16, "2 chunks vs 1")


@pytest.mark.parametrize("fp16_recurrence", [False, True])
def test_amp_training_loop_of_the_reference(fp16_recurrence):
    """The shape of the reference's own AMP test (test/test_amp.py:42-82): one SRUCell 304 -> 304, input
    rand(304, 200, 304), fp16 autocast, loss = h.sum(), GradScaler + Adam, a few iterations.  Gradients of the
    first iteration against the oracle; every later loss finite and the scaler never skips a step."""
    from sru_b200.modules import SRUCell
    torch.manual_seed(1)
    cell = SRUCell(304, 304, amp_recurrence_fp16=fp16_recurrence).to(DEV)
    x = torch.rand(304, 200, 304, generator=torch.Generator().manual_seed(2)).to(DEV)
    opt = torch.optim.Adam(cell.parameters(), lr=0.02)
    scaler = torch.amp.GradScaler("cuda", init_scale=128.0)
    from oracle.ref_model import OracleSRU
    ref = OracleSRU(304, 304, num_layers=1, rescale=True)
    with torch.no_grad():
        for n, p in cell.named_parameters():
            q = dict(ref.rnn_lst[0].named_parameters())[n]
            q.copy_(p.detach().cpu().half().float() if n == "weight" else p.detach().cpu())
        ref.rnn_lst[0].scale_x.copy_(cell.scale_x.cpu())
    rows = [0, 77, 199]
    oh, _ = ref(x[:, rows].cpu().half().float())
    oh.sum().backward()
    name = "test_amp/fp16_recurrence=%d" % fp16_recurrence
    for it in range(4):
        with torch.autocast("cuda", dtype=torch.float16):
            h, c = cell(x)
            s = h.sum()
        assert h.dtype == (torch.float16 if fp16_recurrence else torch.float32)
        opt.zero_grad()
        scaler.scale(s).backward()
        if it == 0:
            check_parity(name, "h", h[:, rows], oh.detach(), TOL16, "3 rows")
        for n, p in cell.named_parameters():        # fp32 master gradients (the weight's straight from the GEMM)
            assert p.grad is not None and p.grad.dtype == torch.float32, (it, n)
        scaler.step(opt)                            # skips the step if a half-precision gradient overflowed
        scaler.update()
        assert torch.isfinite(s.float())


def test_packed_sequence_compat_return_and_input_projection_on_gpu():
    """PackedSequence input, nn.RNN-style state layout and proj_input_to_hidden_first on the CUDA path
    (sru/modules.py:593-604, :638-646, :520-528), fp32, against the oracle model."""
    from torch.nn.utils.rnn import pack_padded_sequence, pad_packed_sequence
    SRU = _sru()
    torch.manual_seed(3)
    model = SRU(6, 8, num_layers=2, bidirectional=True, proj_input_to_hidden_first=True,
                nn_rnn_compatible_return=True, rescale=True).to(DEV).eval()
    lens = torch.tensor([7, 5, 5, 2])
    x = torch.randn(7, 4, 6, generator=torch.Generator().manual_seed(8))
    ref = to_oracle(model).eval()
    with torch.no_grad():
        hp, c = model(pack_padded_sequence(x.to(DEV), lens))
        ohp, oc = ref(pack_padded_sequence(x, lens))
    h, hl = pad_packed_sequence(hp)
    oh, ohl = pad_packed_sequence(ohp)
    assert c.shape == (4, 4, 8) and torch.equal(hl, ohl)
    check_parity("packed_compat_in2hid", "h", h, oh, 1e-5)
    check_parity("packed_compat_in2hid", "c", c, oc, 1e-5)
