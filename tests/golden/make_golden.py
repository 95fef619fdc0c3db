"""Generate the golden vectors under tests/golden/ from the REFERENCE implementation.

Run where the reference checkout is importable (it is not needed at test time):

    SRU_REFERENCE_ROOT=<reference checkout> python tests/golden/make_golden.py

What is recorded
* ``op_cases.pt``    -- inputs/outputs/gradients of the reference's
  ``sru.ops.elementwise_recurrence_naive`` (sru/ops.py:146-250, autograd for the
  gradients), computed in float64, for a sweep of small shapes covering
  uni/bi, k=3/4, no-skip, mask_pad, mask_c, c0 != 0, scale_x, custom V, tanh.
* ``model_cases.pt`` -- reference ``sru.SRU`` on CPU (float32): state_dict, input,
  outputs and parameter gradients for the shapes of the reference's own tests
  (test/sru/test_sru.py:128-162, test/sru/test_torchscript.py:6-53) and for the
  first benchmark configuration (2 layers, 128 -> 128, L=20, B=32).
* ``regression_2_3_5.pt`` -- the tensors of the reference's regression artifact
  test/regression/artifacts/2.3.5.pt (its test: test/regression/test_regression.py:19-51),
  re-saved as a plain dict of tensors.
* ``layer_norm_cases.pt`` -- the layer normalisation of a reference ``sru.SRUCell`` (the ``nn.LayerNorm``
  it constructs at sru/modules.py:155-160 and calls at :252-253 / :278-279), float64, random affine
  parameters: input, output, and the gradients autograd gives for input, weight and bias.

``python tests/golden/make_golden.py layer_norm`` regenerates only the last file.
"""
import os
import sys
import warnings

import torch

_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.environ.get("SRU_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO), "reference"))
os.environ.setdefault("TORCH_EXTENSIONS_DIR", "/tmp/sru_ref_torch_ext")
sys.path.insert(0, REF)
warnings.filterwarnings("ignore")
import sru  # noqa: E402  (the reference package)
from sru.ops import elementwise_recurrence_naive  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def op_case(name, L, B, d, bidirectional, k, has_skip, mask_pad, mask_c, c0, scale, custom, act, seed):
    g = torch.Generator().manual_seed(seed)
    dirs = 2 if bidirectional else 1
    D = d * dirs
    dt = torch.float64
    U = torch.randn(L, B, D * k, generator=g, dtype=dt, requires_grad=True)
    x = torch.randn(L, B, D, generator=g, dtype=dt, requires_grad=True)
    if custom:
        wc = torch.randn(L, B, D * 2, generator=g, dtype=dt, requires_grad=True)
    else:
        wc = torch.randn(2 * D, generator=g, dtype=dt, requires_grad=True)
    bias = torch.randn(2 * D, generator=g, dtype=dt, requires_grad=True)
    cinit = (torch.randn(B, D, generator=g, dtype=dt) if c0 else torch.zeros(B, D, dtype=dt)).requires_grad_(True)
    mc = None
    if mask_c:
        mc = (torch.rand(B, D, generator=g, dtype=dt) > 0.3).to(dt) / 0.7
    mp = None
    if mask_pad == "tail":
        lens = torch.randint(max(1, L // 2), L + 1, (B,), generator=g)
        mp = (torch.arange(L).view(L, 1) >= lens.view(1, B))
    elif mask_pad == "random":
        mp = torch.rand(L, B, generator=g) > 0.6
    sx = None if scale is None else torch.tensor([scale], dtype=dt)
    gh = torch.randn(L, B, D, generator=g, dtype=dt)
    gl = torch.randn(B, D, generator=g, dtype=dt)
    h, c_last = elementwise_recurrence_naive(U, x, wc, bias, cinit, act, d, bidirectional, has_skip,
                                             sx, mc, mp)
    loss = (h * gh).sum() + (c_last * gl).sum()
    loss.backward()
    use_x = has_skip and k == 3
    return {
        "name": name,
        "meta": dict(L=L, B=B, d=d, dirs=dirs, k=k, has_skip=has_skip, custom=custom, act=act,
                     scale=scale),
        "U": U.detach(), "x": x.detach(), "weight_c": wc.detach(), "bias": bias.detach(),
        "c_init": cinit.detach(), "mask_c": mc, "mask_pad": mp, "grad_h": gh, "grad_last": gl,
        "h": h.detach(), "c_last": c_last.detach(),
        "grad_U": U.grad, "grad_x": x.grad if use_x else None, "grad_weight_c": wc.grad,
        "grad_bias": bias.grad, "grad_c_init": cinit.grad,
    }


def make_op_cases():
    cases = []
    s = 100

    def add(*a, **kw):
        nonlocal s
        s += 1
        cases.append(op_case(*a, seed=s, **kw))

    #    name                L  B  d  bi     k  skip  mask_pad  mask_c c0     scale custom act
    add("uni_k3_simple",     5, 3, 8, False, 3, True, None,     False, False, None, False, 0)
    add("uni_k3_c0_scale",   6, 2, 8, False, 3, True, None,     False, True,  1.7,  False, 0)
    add("bi_k3_all",         7, 3, 8, True,  3, True, "tail",   True,  True,  1.3,  False, 0)
    add("bi_k3_randpad",     9, 4, 4, True,  3, True, "random", True,  True,  None, False, 0)
    add("uni_k4_pad",        6, 3, 8, False, 4, True, "tail",   False, True,  None, False, 0)
    add("bi_k4_maskc",       5, 2, 16, True, 4, True, "random", True,  True,  None, False, 0)
    add("uni_noskip",        5, 3, 8, False, 3, False, "tail",  True,  True,  None, False, 0)
    add("bi_noskip",         4, 2, 8, True,  3, False, None,    False, False, None, False, 0)
    add("uni_custom_v",      5, 2, 8, False, 3, True, "tail",   True,  True,  1.2,  True,  0)
    add("bi_custom_v_k4",    4, 3, 4, True,  4, True, "random", False, True,  None, True,  0)
    add("uni_tanh",          5, 2, 8, False, 3, True, None,     True,  True,  None, False, 1)
    add("bi_tanh_k4",        6, 2, 4, True,  4, True, "tail",   True,  True,  None, False, 1)
    add("uni_odd_d7",        4, 3, 7, False, 3, True, "tail",   True,  True,  1.1,  False, 0)
    add("bi_odd_d3",         5, 5, 3, True,  3, True, "random", False, True,  None, False, 0)
    add("uni_L1",            1, 4, 8, False, 3, True, None,     False, True,  None, False, 0)
    add("bi_L1_pad",         1, 4, 8, True,  4, True, "random", True,  True,  None, False, 0)
    add("uni_L37_d16",       37, 2, 16, False, 3, True, "tail", True,  True,  1.5,  False, 0)
    add("bi_L33_d16",        33, 3, 16, True, 3, True, "tail",  True,  True,  None, False, 0)
    add("bi_L19_d16_k4",     19, 2, 16, True, 4, True, "random", True, True,  None, False, 0)
    torch.save(cases, os.path.join(OUT, "op_cases.pt"))
    print("op_cases:", len(cases))


def model_case(name, kwargs, L, B, seed, mask=False, loss="sum", c0=False, train=True):
    torch.manual_seed(seed)
    model = sru.SRU(**kwargs)
    model.train(train)
    g = torch.Generator().manual_seed(1000 + seed)
    x = torch.randn(L, B, kwargs["input_size"], generator=g)
    mp = None
    if mask:
        lens = torch.randint(max(1, L // 2), L + 1, (B,), generator=g)
        mp = (torch.arange(L).view(L, 1) >= lens.view(1, B))
    c0_t = None
    if c0:
        dirs = 2 if kwargs.get("bidirectional") else 1
        c0_t = torch.randn(kwargs.get("num_layers", 2), B, kwargs["hidden_size"] * dirs, generator=g)
    state = {k_: v.clone() for k_, v in model.state_dict().items()}
    h, c = model(x, c0_t, mask_pad=mp)
    (h.sum() if loss == "sum" else (h ** 2).mean()).backward()
    grads = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    return {"name": name, "kwargs": kwargs, "loss": loss, "state": state, "x": x, "mask_pad": mp,
            "c0": c0_t, "h": h.detach(), "c": c.detach(), "grads": grads}


def make_model_cases():
    cases = []
    i = 0
    for bi in (False, True):
        for ln in (False, True):
            for na in (False, True):
                i += 1
                cases.append(model_case(
                    "test_sru_backward_bi%d_ln%d_na%d" % (bi, ln, na),
                    dict(input_size=4, hidden_size=2, bidirectional=bi, layer_norm=ln,
                         normalize_after=na), 3, 5, 123 + i))
    for bi in (False, True):
        for proj in (0, 4):
            i += 1
            cases.append(model_case(
                "torchscript_shape_bi%d_proj%d" % (bi, proj),
                dict(input_size=32, hidden_size=32, num_layers=2, bidirectional=bi, rescale=True,
                     projection_size=proj, layer_norm=bool(proj)), 16, 8, 200 + i, mask=bi, c0=True))
    cases.append(model_case(
        "config1", dict(input_size=128, hidden_size=128, num_layers=2, dropout=0.0,
                        highway_bias=-2.0, layer_norm=False), 20, 32, 0))
    cases.append(model_case(
        "noskip_tanh", dict(input_size=8, hidden_size=8, num_layers=2, has_skip_term=False,
                            use_tanh=True), 6, 3, 301, mask=True))
    cases.append(model_case(
        "in2hid_compat", dict(input_size=6, hidden_size=8, num_layers=2, bidirectional=True,
                              proj_input_to_hidden_first=True, nn_rnn_compatible_return=True,
                              highway_bias=-1.0, rescale=True), 5, 3, 302, loss="sq"))
    torch.save(cases, os.path.join(OUT, "model_cases.pt"))
    print("model_cases:", len(cases))


def make_regression():
    art = torch.load(os.path.join(REF, "test/regression/artifacts/2.3.5.pt"), weights_only=False)
    out = {
        "version": art["sru.__version__"],
        "kwargs": art["sru_kwargs"],
        "state": {k_: v.clone() for k_, v in art["model_state"].items()},
        "x": art["inputs"].clone(),
        "h": art["outputs"][0].clone(),
        "c": art["outputs"][1].clone(),
    }
    torch.save(out, os.path.join(OUT, "regression_2_3_5.pt"))
    print("regression artifact:", out["version"], out["kwargs"])


def make_layer_norm_cases():
    cases = []
    for i, (rows_shape, n, after) in enumerate([((7, 3), 8, False), ((9,), 120, False), ((2, 2), 512, False),
                                                ((3,), 1024, True), ((1, 2), 2048, True), ((2,), 4096, True),
                                                ((6, 2), 24, False), ((2,), 1000, False)]):
        g = torch.Generator().manual_seed(900 + i)
        hidden = n if not after else n
        cell = sru.SRUCell(n if not after else 8, hidden, layer_norm=True, normalize_after=after).double()
        ln = cell.layer_norm
        assert isinstance(ln, torch.nn.LayerNorm) and ln.normalized_shape == (n,)
        with torch.no_grad():
            ln.weight.copy_(torch.randn(n, generator=g, dtype=torch.float64) * 0.5 + 1.0)
            ln.bias.copy_(torch.randn(n, generator=g, dtype=torch.float64) * 0.3)
        x = (torch.randn(*rows_shape, n, generator=g, dtype=torch.float64) * 1.7 + 0.4).requires_grad_(True)
        dy = torch.randn(*rows_shape, n, generator=g, dtype=torch.float64)
        y = ln(x)
        y.backward(dy)
        cases.append({"n": n, "eps": ln.eps, "x": x.detach().clone(), "weight": ln.weight.detach().clone(),
                      "bias": ln.bias.detach().clone(), "dy": dy, "y": y.detach().clone(),
                      "dx": x.grad.clone(), "dweight": ln.weight.grad.clone(), "dbias": ln.bias.grad.clone()})
    torch.save(cases, os.path.join(OUT, "layer_norm_cases.pt"))
    print("layer_norm_cases:", len(cases))


if __name__ == "__main__":
    if sys.argv[1:] == ["layer_norm"]:
        make_layer_norm_cases()
    else:
        make_op_cases()
        make_model_cases()
        make_regression()
        make_layer_norm_cases()
