"""Batch-sharded data parallelism on CPU ranks (gloo, world size 2): the per-layer gradient
all-reducer must reproduce the single-process gradients of the full batch.  The layers compute
with the CPU oracle model (the product path has no CPU execution); what is under test is the
host logic: sharding, bucket views, hook-driven asynchronous all-reduce, loss normalisation."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.ref_model import OracleSRU
from sru_b200.distributed import LayerGradAllReducer, shard_batch, use_global_dropout_masks

KW = dict(input_size=12, hidden_size=8, num_layers=3, bidirectional=True, layer_norm=True, rescale=True)
L, B = 7, 5   # odd batch: ranks get 3 and 2 sequences


def _inputs():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(L, B, KW["input_size"], generator=g)
    lens = torch.randint(3, L + 1, (B,), generator=g)
    mask = torch.arange(L).view(L, 1) >= lens.view(1, B)
    return x, mask


def _model(dropout=0.0):
    torch.manual_seed(7)
    kw = dict(KW, dropout=dropout)
    return OracleSRU(kw.pop("input_size"), kw.pop("hidden_size"), **kw).train()


def _global_masks(model, rank, world):
    """Dropout masks drawn for the global batch, identically on every rank (the oracle model asks its
    ``mask_source``; the shipped layers ask ``get_dropout_mask_``, which is what the call installs)."""
    use_global_dropout_masks(model, B, rank, world, seed=11)
    model.mask_source = lambda li, like, size, p: model.rnn_lst[li].get_dropout_mask_(size, p)


def _loss(h):
    return (h ** 2).sum() / float(L * B * h.size(-1))   # normalised by the GLOBAL token count


def _worker(rank, world, port, out, mode):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    model = _model(dropout=0.3 if mode == "global_dropout" else 0.0)
    if mode == "global_dropout":
        _global_masks(model, rank, world)
    x, mask = _inputs()
    xs, ms = shard_batch(x, rank, world), shard_batch(mask, rank, world)
    reducer = LayerGradAllReducer(model, reduce_dtype=torch.bfloat16 if mode == "bf16_wire" else None)
    assert len(reducer.buckets) == KW["num_layers"]
    if mode == "frozen_param":
        # a parameter that never receives a gradient must not hold back its layer's all-reduce
        model.rnn_lst[1].weight_c.requires_grad_(False)
        reducer.remove()
        reducer = LayerGradAllReducer(model)
    opt = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=0.0)
    raised = False
    for step in range(3):                    # later steps check zeroing / re-arming
        if mode == "optimizer_zero_grad":
            opt.zero_grad(set_to_none=True)  # detaches every p.grad from its bucket
        elif mode == "no_zero_grad_rearm" and step > 0:
            for b in reducer.buckets:        # zeroed by hand; finish() alone must have re-armed the reducer
                b.zero_()
        else:
            reducer.zero_grad()
        h, c = model(xs, mask_pad=ms)
        _loss(h).backward()
        if mode == "double_backward" and step == 0:
            h, c = model(xs, mask_pad=ms)
            try:
                _loss(h).backward()
            except RuntimeError as e:
                raised = "second gradient" in str(e)
        reducer.finish()
        for n, p in model.named_parameters():
            if p.requires_grad:
                assert p.grad.data_ptr() == reducer._views[id(p)].data_ptr(), n     # views of the buckets again
    if mode == "double_backward":
        assert raised
    if rank == 0:
        torch.save({n: p.grad.clone() for n, p in model.named_parameters() if p.requires_grad}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_shard_batch_covers_everything():
    x = torch.arange(2 * 7 * 3).view(2, 7, 3)
    parts = [shard_batch(x, r, 3) for r in range(3)]
    assert [p.size(1) for p in parts] == [3, 2, 2]
    assert torch.equal(torch.cat(parts, 1), x)
    assert shard_batch(None, 0, 2) is None


@pytest.mark.parametrize("mode", ["plain", "optimizer_zero_grad", "no_zero_grad_rearm", "double_backward",
                                  "frozen_param", "bf16_wire", "global_dropout"])
def test_two_rank_gradients_equal_single_process(tmp_path, mode):
    """Gradients after three steps on two ranks equal the single-process gradients of the whole batch:
    with the reducer's own zero_grad; with an optimizer's zero_grad(set_to_none=True), which detaches the
    gradients from the buckets; when only finish() re-arms the reducer; after a refused second backward;
    with a parameter that receives no gradient; with the sum taken on a bf16 copy of the bucket; with dropout
    masks drawn for the global batch (every rank keeps its rows of the same mask, so the sharded step computes
    what the single process computes)."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "grads.pt")
    mp.spawn(_worker, args=(2, port, out, mode), nprocs=2, join=True)
    got = torch.load(out)
    model = _model(dropout=0.3 if mode == "global_dropout" else 0.0)
    x, mask = _inputs()
    if mode == "global_dropout":
        _global_masks(model, 0, 1)
        for _ in range(2):                  # the workers' third step uses each layer's third draw
            model(x, mask_pad=mask)
    h, c = model(x, mask_pad=mask)
    _loss(h).backward()
    named = dict(model.named_parameters())
    assert len(got) >= len(named) - 1
    for n, g in got.items():
        if mode == "bf16_wire":
            assert torch.allclose(g, named[n].grad, rtol=2e-2, atol=1e-4), n
        elif mode == "double_backward":
            continue    # step 0 was disturbed on purpose; the later steps were checked inside the worker
        else:
            assert torch.allclose(g, named[n].grad, rtol=1e-4, atol=1e-6), n
