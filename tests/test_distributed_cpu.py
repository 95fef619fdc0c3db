"""Batch-sharded data parallelism on CPU ranks (gloo, world size 2): the per-layer gradient
all-reducer must reproduce the single-process gradients of the full batch.  The layers compute
with the CPU oracle model (the product path has no CPU execution); what is under test is the
host logic: sharding, bucket views, hook-driven asynchronous all-reduce, loss normalisation."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.cpu_model import to_oracle
from sru_b200.distributed import LayerGradAllReducer, shard_batch
from sru_b200.modules import SRU

KW = dict(input_size=12, hidden_size=8, num_layers=3, bidirectional=True, layer_norm=True, rescale=True)
L, B = 7, 5   # odd batch: ranks get 3 and 2 sequences


def _inputs():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(L, B, KW["input_size"], generator=g)
    lens = torch.randint(3, L + 1, (B,), generator=g)
    mask = torch.arange(L).view(L, 1) >= lens.view(1, B)
    return x, mask


def _model():
    torch.manual_seed(7)
    return to_oracle(SRU(**KW)).train()


def _loss(h):
    return (h ** 2).sum() / float(L * B * h.size(-1))   # normalised by the GLOBAL token count


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    model = _model()
    x, mask = _inputs()
    xs, ms = shard_batch(x, rank, world), shard_batch(mask, rank, world)
    reducer = LayerGradAllReducer(model)
    assert len(reducer.buckets) == KW["num_layers"]
    for _ in range(2):                       # second step checks zero_grad / re-arming
        reducer.zero_grad()
        h, c = model(xs, mask_pad=ms)
        _loss(h).backward()
        reducer.finish()
    if rank == 0:
        torch.save({n: p.grad.clone() for n, p in model.named_parameters()}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_shard_batch_covers_everything():
    x = torch.arange(2 * 7 * 3).view(2, 7, 3)
    parts = [shard_batch(x, r, 3) for r in range(3)]
    assert [p.size(1) for p in parts] == [3, 2, 2]
    assert torch.equal(torch.cat(parts, 1), x)
    assert shard_batch(None, 0, 2) is None


def test_two_rank_gradients_equal_single_process(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "grads.pt")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = torch.load(out)
    model = _model()
    x, mask = _inputs()
    h, c = model(x, mask_pad=mask)
    _loss(h).backward()
    for n, p in model.named_parameters():
        assert torch.allclose(got[n], p.grad, rtol=1e-4, atol=1e-6), n
