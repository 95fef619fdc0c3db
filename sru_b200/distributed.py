"""Batch-sharded data parallelism for SRU training: one process per GPU, parameters replicated,
the batch dimension (dim 1 of (length, batch, features)) split across ranks, parameter
gradients summed with one all-reduce per layer.

The reference has no distributed code (its only multi-GPU artefact scatters the batch
dimension with nn.DataParallel in misc/test_multigpu.py:43-44); sequences are independent, so
nothing but the parameter gradients ever crosses ranks.

``LayerGradAllReducer`` keeps each layer's gradients in one flat bucket (``p.grad`` are views
of it), and starts that layer's all-reduce asynchronously as soon as autograd has produced the
last gradient of the layer, so the collective of layer i overlaps the backward of layers < i.
Works with any ``torch.distributed`` backend (NCCL on GPUs, gloo in the CPU tests).
"""
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


def shard_batch(t: Optional[torch.Tensor], rank: int, world: int, dim: int = 1) -> Optional[torch.Tensor]:
    """This rank's contiguous slice of the batch dimension (sizes differ by at most one)."""
    if t is None:
        return None
    n = t.size(dim)
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return t.narrow(dim, start, base + (1 if rank < rem else 0)).contiguous()


class LayerGradAllReducer:
    """Per-layer bucketed gradient all-reduce (SUM) overlapped with backward.

    groups: list of lists of parameters; by default one group per child of ``model.rnn_lst``
    plus one group for whatever is left.  Call ``finish()`` after ``backward()`` and before the
    gradients are read.
    """

    def __init__(self, model: nn.Module, process_group=None, groups: Optional[List[List[nn.Parameter]]] = None):
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        if self.world > 1:
            # the all-reduces run next to backward and take SMs from it for a while: let the persistent GEMM hand
            # out its tiles dynamically so that pairs that start late simply take fewer (explicit settings win)
            os.environ.setdefault("SRU_B200_GEMM_DYNAMIC", "1")
        if groups is None:
            groups = []
            seen = set()
            for layer in getattr(model, "rnn_lst", []):
                ps = [p for p in layer.parameters() if p.requires_grad]
                seen.update(id(p) for p in ps)
                if ps:
                    groups.append(ps)
            rest = [p for p in model.parameters() if p.requires_grad and id(p) not in seen]
            if rest:
                groups.append(rest)
        self.groups = groups
        self.buckets: List[torch.Tensor] = []
        self._pending: List[int] = []
        self._handles = []
        self._index: Dict[int, int] = {}
        self._hooks = []
        for gi, ps in enumerate(groups):
            total = sum(p.numel() for p in ps)
            flat = torch.zeros(total, dtype=ps[0].dtype, device=ps[0].device)
            off = 0
            for p in ps:
                if p.dtype != flat.dtype:
                    raise ValueError("all parameters of a bucket must share one dtype")
                p.grad = flat[off:off + p.numel()].view_as(p)
                off += p.numel()
                self._index[id(p)] = gi
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))
            self.buckets.append(flat)
            self._pending.append(len(ps))

    def zero_grad(self):
        """Zeroes the buckets in place (gradients stay views of them) and re-arms the counters."""
        for gi, flat in enumerate(self.buckets):
            flat.zero_()
            self._pending[gi] = len(self.groups[gi])
        self._handles = []

    def _on_grad(self, p: torch.Tensor):
        gi = self._index[id(p)]
        self._pending[gi] -= 1
        if self._pending[gi] == 0 and self.world > 1:
            self._handles.append(dist.all_reduce(self.buckets[gi], op=dist.ReduceOp.SUM, group=self.group,
                                                 async_op=True))

    def finish(self):
        """Waits for every all-reduce started during backward (stream-ordered for NCCL)."""
        for h in self._handles:
            h.wait()
        self._handles = []

    def bytes_per_step(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.buckets)

    def remove(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []
