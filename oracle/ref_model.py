"""CPU restatement of the reference's layer stack around the scan.  TEST INFRASTRUCTURE ONLY.

``OracleSRU`` is a self-contained model: it shares no code with the shipped package (it does not
import it), so the residual / layer-norm order, the dropout placement, the ``c0`` split, the
low-rank chain and the return conventions are checked against an independent statement of what
the reference does.  What it follows, by function:

* parameter shapes and names            sru/modules.py:126-160 (SRUCell.__init__), :520-570 (SRU.__init__)
* ``init_like_reference``               sru/modules.py:164-233 (SRUCell.reset_parameters; same order of
                                        random draws, so the same seed gives the same weights)
* ``_layer_forward``                    sru/modules.py:235-281 (SRUCell.forward), :321-378 (compute_UV, compute_U)
* ``forward``                           sru/modules.py:572-652 (SRU.forward)
* dropout mask                          sru/modules.py:380-387

The recurrence is ``sru_oracle.elementwise_recurrence_oracle`` (the C restatement of the scan, with
the casts of sru/ops.py:116-127: always float32, or float64 for float64 tensors) and the layer
normalisation is ``sru_oracle.layer_norm_oracle``.  Pinned by tests/test_oracle.py against the golden
vectors recorded from the reference's own ``sru.SRU`` (tests/golden/model_cases.pt).
"""
import copy
import math
from typing import Callable, Dict, List, Optional

import torch
import torch.nn as nn
from torch.nn.utils.rnn import PackedSequence, pack_padded_sequence, pad_packed_sequence

from . import sru_oracle

_DEFAULTS = dict(num_layers=2, dropout=0.0, rnn_dropout=0.0, bidirectional=False, projection_size=0,
                 use_tanh=False, layer_norm=False, highway_bias=0.0, has_skip_term=True, rescale=False,
                 v1=False, nn_rnn_compatible_return=False, custom_m=None, proj_input_to_hidden_first=False,
                 amp_recurrence_fp16=False, normalize_after=False, weight_c_init=None)


class _Norm(nn.Module):
    """Holder of a layer normalisation's affine parameters (names as nn.LayerNorm's)."""

    def __init__(self, n: int):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n))
        self.bias = nn.Parameter(torch.zeros(n))
        self.eps = 1e-5


class _Layer(nn.Module):
    """Parameters and static facts of one layer; registration order = the reference's."""

    def __init__(self, n_in: int, d: int, dirs: int, dropout: float, rnn_dropout: float, proj: int, tanh: bool,
                 layer_norm: bool, highway_bias: float, has_skip: bool, rescale: bool, v1: bool, custom_m,
                 normalize_after: bool, weight_c_init):
        super().__init__()
        self.n_in, self.d, self.dirs, self.D = n_in, d, dirs, d * dirs
        self.p_drop, self.p_rnn_drop = float(dropout), float(rnn_dropout)
        self.act = 1 if tanh else 0
        self.highway_bias, self.has_skip, self.rescale, self.v1 = highway_bias, has_skip, rescale, v1
        self.normalize_after, self.weight_c_init = normalize_after, weight_c_init
        self.custom_m = custom_m
        self.proj = proj if 0 < proj < min(n_in, self.D) else 0
        self.k = 4 if (has_skip and n_in != self.D) else 3
        if custom_m is None:
            if self.proj:
                self.weight_proj = nn.Parameter(torch.empty(n_in, self.proj))
                self.weight = nn.Parameter(torch.empty(self.proj, self.D * self.k))
            else:
                self.weight_proj = None
                self.weight = nn.Parameter(torch.empty(n_in, self.D * self.k))
        self.weight_c = nn.Parameter(torch.empty(2 * self.D))
        self.bias = nn.Parameter(torch.empty(2 * self.D))
        self.register_buffer("scale_x", torch.zeros(1))
        self.layer_norm = _Norm(self.D if normalize_after else n_in) if layer_norm else None

    @torch.no_grad()
    def init_like_reference(self):
        D, hb = self.D, self.highway_bias
        s_highway = math.sqrt(1.0 + 2.0 * math.exp(hb))
        self.bias.zero_()
        self.bias[D:] = hb
        self.scale_x[0] = s_highway if (self.rescale and self.has_skip) else 1.0
        w4 = None
        if self.custom_m is None:
            rows = self.weight.size(0)
            r = math.sqrt(3.0 / rows)
            self.weight.uniform_(-r, r)
            if self.proj:
                r = math.sqrt(3.0 / self.weight_proj.size(0))
                self.weight_proj.uniform_(-r, r)
            w4 = self.weight.view(rows, self.dirs, self.d, self.k)        # gate index innermost
            if self.p_drop > 0:
                w4[..., 0] *= math.sqrt(1.0 - self.p_drop)
            if self.p_rnn_drop > 0:
                w4 *= math.sqrt(1.0 - self.p_rnn_drop)
            if self.layer_norm is not None:
                w4 *= 0.1
            if self.rescale and self.has_skip and self.k == 4:
                w4[..., 3] *= s_highway
        elif hasattr(self.custom_m, "reset_parameters"):
            self.custom_m.reset_parameters()
        if self.v1:
            self.weight_c.zero_()
            self.weight_c.requires_grad = False
            return
        if self.weight_c_init is None:
            self.weight_c.uniform_(-math.sqrt(3.0), math.sqrt(3.0))
            self.weight_c *= math.sqrt(0.5)
        else:
            self.weight_c.uniform_(-self.weight_c_init, self.weight_c_init)
        if w4 is not None:
            w4[..., 1] *= math.sqrt(0.5)
            w4[..., 2] *= math.sqrt(0.5)


def _default_mask(layer_index: int, like: torch.Tensor, size, p: float) -> torch.Tensor:
    return like.new_empty(size).bernoulli_(1 - p).div_(1 - p)


class OracleSRU(nn.Module):
    """Stack of SRU layers on the CPU.  ``kwargs`` are the reference's ``sru.SRU`` constructor arguments.

    ``mask_source(layer_index, like, size, p)`` supplies dropout masks (default: drawn the way the reference
    draws them); tests that compare with a GPU run replay the GPU's masks through it.
    """

    def __init__(self, input_size: int, hidden_size: int, **kw):
        super().__init__()
        unknown = set(kw) - set(_DEFAULTS)
        if unknown:
            raise TypeError("unknown SRU arguments: %s" % sorted(unknown))
        o = dict(_DEFAULTS)
        o.update(kw)
        self.opts = o
        self.input_size, self.hidden_size = input_size, hidden_size
        self.dirs = 2 if o["bidirectional"] else 1
        self.D = hidden_size * self.dirs
        self.num_layers = o["num_layers"]
        self.input_to_hidden = None
        first_in = input_size
        if o["proj_input_to_hidden_first"] and input_size != self.D:
            first_in = self.D
            self.input_to_hidden = nn.Linear(input_size, self.D, bias=False)
        layers = []
        for i in range(self.num_layers):
            cm = o["custom_m"]
            if cm is not None:
                cm = cm[i] if isinstance(cm, list) else copy.deepcopy(cm)
            layer = _Layer(first_in if i == 0 else self.D, hidden_size, self.dirs,
                           o["dropout"] if i + 1 != self.num_layers else 0.0, o["rnn_dropout"],
                           o["projection_size"], o["use_tanh"], o["layer_norm"], o["highway_bias"],
                           o["has_skip_term"], o["rescale"], o["v1"], cm, o["normalize_after"],
                           o["weight_c_init"])
            layer.init_like_reference()
            layers.append(layer)
        self.rnn_lst = nn.ModuleList(layers)
        self.mask_source: Callable = _default_mask
        # (U, x, V, bias, c0, activation_type, d, bidirectional, has_skip, scale_x, mask_c, mask_pad) -> (h, c_last);
        # the benchmark's forward-only CPU baseline puts the reference's compiled operator here
        self.recurrence: Callable = sru_oracle.elementwise_recurrence_oracle
        # 16-bit checks: the oracle of a 16-bit run is the float32 recurrence fed the same 16-bit-rounded U, as the
        # parity metric defines it (gradients stay unrounded)
        self.round_u_to: Optional[torch.dtype] = None

    # ---- one layer: sru/modules.py:235-281 ----
    def _layer_forward(self, li: int, lay: _Layer, inp: torch.Tensor, c0: Optional[torch.Tensor],
                       mask_pad: Optional[torch.Tensor]):
        if inp.dim() not in (2, 3):
            raise ValueError("Input must be 2 or 3 dimensional")
        nb = inp.size(-2)
        if c0 is None:
            c0 = torch.zeros(nb, lay.D, dtype=inp.dtype)
        skip_input = inp
        real = torch.float64 if inp.dtype == torch.float64 else torch.float32
        if lay.layer_norm is not None and not lay.normalize_after:
            inp = sru_oracle.layer_norm_oracle(inp.to(real), lay.layer_norm.weight, lay.layer_norm.bias,
                                               lay.layer_norm.eps)
        if self.training and lay.p_rnn_drop > 0:
            inp = inp * self.mask_source(li, lay.bias.data, (nb, inp.size(-1)), lay.p_rnn_drop).expand_as(inp)
        scale = lay.scale_x if lay.rescale else None
        mask_c = None
        if self.training and lay.p_drop > 0:
            mask_c = self.mask_source(li, lay.bias.data, (nb, lay.D), lay.p_drop)
        # U (and the optional per-step V of a custom module): sru/modules.py:321-378
        if lay.custom_m is None:
            flat = inp if inp.dim() == 2 else inp.contiguous().view(-1, lay.n_in)
            U = flat.mm(lay.weight_proj).mm(lay.weight) if lay.weight_proj is not None else flat.mm(lay.weight)
            V = lay.weight_c
        else:
            ret = lay.custom_m(inp)
            if isinstance(ret, (tuple, list)):
                if len(ret) > 2:
                    raise Exception("Custom module must return 1 or 2 tensors but got {}.".format(len(ret)))
                U, V = ret[0], ret[1] + lay.weight_c
            else:
                U, V = ret, lay.weight_c
        if self.round_u_to is not None:
            # forward value only: a 16-bit cast in the autograd graph would also round grad_U, which underflows in
            # fp16 when the oracle runs without the loss scale of the run it checks
            U = U + (U.to(self.round_u_to).to(U.dtype) - U).detach()
        h, c = self.recurrence(
            U.to(real), skip_input.to(real), V.to(real), lay.bias.to(real), c0.to(real), lay.act, lay.d,
            lay.dirs == 2, lay.has_skip, None if scale is None else scale.to(real),
            None if mask_c is None else mask_c.to(real), mask_pad)
        if lay.layer_norm is not None and lay.normalize_after:
            h = sru_oracle.layer_norm_oracle(h, lay.layer_norm.weight, lay.layer_norm.bias, lay.layer_norm.eps)
        return h, c

    # ---- the stack: sru/modules.py:572-652 ----
    def forward(self, input, c0: Optional[torch.Tensor] = None, mask_pad: Optional[torch.Tensor] = None):
        packed = isinstance(input, PackedSequence)
        lengths = None
        if packed:
            input, lengths = pad_packed_sequence(input)
            steps = torch.arange(int(lengths.max())).unsqueeze(1)
            mask_pad = steps >= lengths.unsqueeze(0)
        if input.dim() != 3:
            raise ValueError("There must be 3 dimensions for (length, batch_size, input_size)")
        if c0 is not None and c0.dim() != 3:
            raise ValueError("c0 must be 3 dim (num_layers, batch_size, output_size)")
        x = input if self.input_to_hidden is None else self.input_to_hidden(input)
        finals: List[torch.Tensor] = []
        for li, lay in enumerate(self.rnn_lst):
            x, c = self._layer_forward(li, lay, x, None if c0 is None else c0[li], mask_pad)
            finals.append(c)
        stacked = torch.stack(finals)
        if self.opts["nn_rnn_compatible_return"]:
            nb = input.size(1)
            stacked = stacked.view(self.num_layers, nb, self.dirs, self.hidden_size).transpose(1, 2)
            stacked = stacked.contiguous().view(self.num_layers * self.dirs, nb, self.hidden_size)
        if packed:
            x = pack_padded_sequence(x, lengths, enforce_sorted=False)
        return x, stacked


def sru_kwargs_of(model) -> Dict:
    """Reads the reference-style constructor arguments back from a model object that carries the
    reference's attribute names (the shipped ``SRU`` does); no import of that model's package."""
    cell = model.rnn_lst[0]
    cms = [c.custom_m for c in model.rnn_lst]
    return dict(
        input_size=model.input_size, hidden_size=model.hidden_size, num_layers=model.num_layers,
        dropout=model.dropout, rnn_dropout=model.rnn_dropout, bidirectional=model.bidirectional,
        projection_size=model.projection_size, use_tanh=bool(cell.activation_type),
        layer_norm=model.use_layer_norm, highway_bias=cell.highway_bias, has_skip_term=model.has_skip_term,
        rescale=cell.rescale, v1=cell.v1, nn_rnn_compatible_return=model.nn_rnn_compatible_return,
        custom_m=None if all(c is None for c in cms) else [copy.deepcopy(c).cpu() for c in cms],
        proj_input_to_hidden_first=model.input_to_hidden is not None,
        amp_recurrence_fp16=getattr(model, "amp_recurrence_fp16", False),
        normalize_after=cell.normalize_after, weight_c_init=cell.weight_c_init)


def from_state(kwargs: Dict, state: Dict[str, torch.Tensor], round_to: Optional[torch.dtype] = None) -> OracleSRU:
    """An OracleSRU with the given reference-style constructor arguments and state dict.

    round_to: round every projection weight (``weight``, ``weight_proj``, ``input_to_hidden.weight``) to
    this 16-bit type and back, the way a 16-bit autocast GEMM sees them, and round each layer's U to it before the
    recurrence (the GEMM's output type); the model itself stays float32.
    """
    kw = dict(kwargs)
    m = OracleSRU(kw.pop("input_size"), kw.pop("hidden_size"), **kw)
    own = m.state_dict()
    extra = set(state) - set(own)
    missing = set(own) - set(state)
    # custom modules register their own entries under rnn_lst.<i>.custom_m.*; everything else must match
    assert not {k for k in extra | missing if ".custom_m." not in k}, (sorted(extra), sorted(missing))
    with torch.no_grad():
        for name, t in own.items():
            if name in state:
                src = state[name].detach().cpu().to(t.dtype)
                if round_to is not None and name.rsplit(".", 1)[-1] in ("weight", "weight_proj") \
                        and ".layer_norm." not in name:
                    src = src.to(round_to).to(t.dtype)
                t.copy_(src)
    m.round_u_to = round_to
    return m


def to_oracle(model, round_to: Optional[torch.dtype] = None) -> OracleSRU:
    """CPU oracle twin of a (possibly CUDA) model with the reference's attribute and state-dict names,
    in the same train / eval mode."""
    m = from_state(sru_kwargs_of(model), {k: v for k, v in model.state_dict().items()}, round_to)
    m.train(model.training)
    return m
