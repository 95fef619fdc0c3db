"""A whole training step (forward and backward of a layer stack: layer norm, projection GEMMs, scans, the fused
gradient sum) captured into one CUDA graph and replayed: the launchers make no call that is illegal during stream
capture (no allocation, no synchronisation, no context-binding runtime call once the thread has a context), every
scratch buffer comes from the caller, and tensor maps travel inside the kernel parameters.  The replay must give the
bits of the eager step on the same data (the kernels are deterministic).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _model(**kw):
    from sru_b200.modules import SRU
    torch.manual_seed(21)
    return SRU(**kw).to(DEV).train()


@pytest.mark.parametrize("kw", [
    dict(input_size=64, hidden_size=64, num_layers=3, bidirectional=True, dropout=0.0),
    dict(input_size=64, hidden_size=128, num_layers=2, layer_norm=True, rescale=True, dropout=0.0),
])
def test_training_step_replays_from_a_graph(kw):
    model = _model(**kw)
    L, B = 33, 8
    g = torch.Generator().manual_seed(2)
    x_static = torch.randn(L, B, kw["input_size"], generator=g).to(DEV)
    lens = torch.randint(L // 2, L + 1, (B,), generator=g)
    mask_static = (torch.arange(L).view(L, 1) >= lens.view(1, B)).to(DEV)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            h, c = model(x_static, mask_pad=mask_static)
            loss = (h.float() ** 2).mean() + c.float().sum() * 1e-3
        loss.backward()
        return loss

    # warm-up on a side stream (allocator pools, lazily loaded kernels, cached scalars), as graph capture requires
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            model.zero_grad(set_to_none=True)
            step()
    torch.cuda.current_stream().wait_stream(side)

    model.zero_grad(set_to_none=True)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        loss_static = step()
    params = [p for p in model.parameters() if p.grad is not None]
    assert params, "backward inside the capture produced gradients"

    for trial in range(2):
        x_new = torch.randn(L, B, kw["input_size"], generator=g).to(DEV)
        x_static.copy_(x_new)
        graph.replay()
        torch.cuda.synchronize()
        got_loss = loss_static.clone()
        got = [p.grad.clone() for p in params]
        # the same step eagerly
        saved = [p.grad for p in params]
        for p in params:
            p.grad = None
        ref_loss = step()
        torch.cuda.synchronize()
        assert torch.equal(got_loss, ref_loss), (trial, float(got_loss), float(ref_loss))
        for p, a in zip(params, got):
            assert torch.equal(a, p.grad), trial
        for p, s in zip(params, saved):
            p.grad = s
    from sru_b200 import _lib
    _lib.check_device_error()
