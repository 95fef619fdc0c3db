"""Batch-sharded data parallelism for SRU training: one process per GPU, parameters replicated,
the batch dimension (dim 1 of (length, batch, features)) split across ranks, parameter
gradients summed with one all-reduce per layer.

The reference has no distributed code (its only multi-GPU artefact scatters the batch
dimension with nn.DataParallel in misc/test_multigpu.py:43-44); sequences are independent, so
nothing but the parameter gradients ever crosses ranks.

``LayerGradAllReducer`` keeps each layer's gradients in one flat bucket (``p.grad`` are views
of it) and all-reduces a bucket asynchronously once autograd has produced the last gradient of
that layer, so the collective of layer i overlaps the backward of the layers below it.
Works with any ``torch.distributed`` backend (NCCL on GPUs, gloo in the CPU tests).

When the collective starts matters: a layer's bucket is complete right after its weight-gradient
GEMM, which is exactly when the NEXT layer's backward scan begins, and both the scan and the
all-reduce are bound by HBM bandwidth.  With ``defer_to_scan_end`` (default) a complete bucket
is held until that next backward scan has been enqueued, so that the all-reduce overlaps the
two tensor-bound GEMMs that follow it instead of the scan.
"""
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import ops


def shard_batch(t: Optional[torch.Tensor], rank: int, world: int, dim: int = 1) -> Optional[torch.Tensor]:
    """This rank's contiguous slice of the batch dimension (sizes differ by at most one)."""
    if t is None:
        return None
    n = t.size(dim)
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return t.narrow(dim, start, base + (1 if rank < rem else 0)).contiguous()


def use_global_dropout_masks(model: nn.Module, global_batch: int, rank: int, world: int, seed: int = 0) -> None:
    """Makes the sharded step draw exactly the dropout masks of the single-process step.

    The reference draws a layer's mask for the whole batch (sru/modules.py:380-387).  With the batch split across
    ranks, each rank would draw its own, different numbers, and the sharded step would no longer compute what the
    single-process step computes.  After this call the masks of ALL layers for the GLOBAL batch come from one draw
    per step of a generator that is seeded identically on every rank (seed, number of draws so far), and every
    layer keeps the rows of this rank's shard, so losses and gradients agree across world sizes up to summation
    order.  Also valid at world 1.  Layers whose width or dropout probability differs from the first layer's draw
    their own global mask the same way.
    """
    base, rem = divmod(global_batch, world)
    start = rank * base + min(rank, rem)
    rows = base + (1 if rank < rem else 0)
    cells = list(getattr(model, "rnn_lst", []))
    if not cells:
        return
    width0, p0 = cells[0].bias.numel() // 2, None
    pools: Dict[int, torch.Tensor] = {}          # draw number -> (layers, global batch, width) masks
    draws = [0] * len(cells)

    def full_masks(like, n, width, p, k, salt):
        gen = torch.Generator(device=like.device)
        gen.manual_seed(seed * 1000003 + salt * 10007 + k)
        return like.new_empty((n, global_batch, width)).bernoulli_(1 - p, generator=gen).div_(1 - p)

    for li, cell in enumerate(cells):
        def draw(size, p, _cell=cell, _li=li):
            nonlocal p0
            like = _cell.bias.data
            k = draws[_li]
            draws[_li] += 1
            if size[0] != rows:
                raise ValueError("dropout mask for %d rows requested, this rank's shard has %d" % (size[0], rows))
            if p0 is None:
                p0 = p
            if size[1] != width0 or p != p0:      # an odd layer: its own global draw
                return full_masks(like, 1, size[1], p, k, 1 + _li)[0, start:start + rows].contiguous()
            if k not in pools:
                pools.clear()                     # the previous step's masks are no longer needed
                pools[k] = full_masks(like, len(cells), width0, p0, k, 0)
            return pools[k][_li, start:start + rows]
        cell.get_dropout_mask_ = draw


class LayerGradAllReducer:
    """Per-layer bucketed gradient all-reduce (SUM) overlapped with backward.

    groups: list of lists of parameters; by default one group per child of ``model.rnn_lst``
    plus one group for whatever is left.

    Protocol per step: zero the gradients (``reducer.zero_grad()``, or any optimizer's
    ``zero_grad`` -- with ``set_to_none=True`` the next backward's fresh gradient tensors are copied
    into the buckets and re-bound as views), run ONE ``backward()``, call ``finish()``, read the
    gradients.  ``finish()`` all-reduces every bucket that backward did not complete (a layer with
    a parameter that received no gradient), waits for all of them and re-arms the reducer.  A second
    ``backward()`` before ``finish()`` raises: its gradients would be added to sums that other ranks
    have already reduced.

    reduce_dtype: all-reduce a copy of the bucket in this dtype (e.g. ``torch.bfloat16``: half the
    bytes on the wire and in HBM) and write the result back into the fp32 bucket; ``None`` reduces
    the bucket itself.
    dynamic_gemm_order: switch the pair GEMM of this package to its dynamic tile order (option
    ``gemm_dynamic``), which keeps a product from waiting on the CTA pairs whose SMs the
    collective held for a while.  Only touched when the world size is above one and the
    parameters live on a GPU.
    """

    def __init__(self, model: nn.Module, process_group=None, groups: Optional[List[List[nn.Parameter]]] = None,
                 reduce_dtype: Optional[torch.dtype] = None, defer_to_scan_end: bool = True,
                 dynamic_gemm_order: bool = True):
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.reduce_dtype = reduce_dtype
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
        self._views: Dict[int, torch.Tensor] = {}      # id(param) -> its slice of the bucket, shaped like the param
        self._index: Dict[int, int] = {}
        self._seen: List[set] = []
        self._launched: List[bool] = []
        self._ready: List[int] = []                     # complete buckets waiting for the next scan backward
        self._handles = []                              # (work handle, bucket index, reduced copy or None)
        self._hooks = []
        on_gpu = False
        for gi, ps in enumerate(groups):
            total = sum(p.numel() for p in ps)
            flat = torch.zeros(total, dtype=ps[0].dtype, device=ps[0].device)
            on_gpu = on_gpu or flat.is_cuda
            off = 0
            for p in ps:
                if p.dtype != flat.dtype:
                    raise ValueError("all parameters of a bucket must share one dtype")
                view = flat[off:off + p.numel()].view_as(p)
                self._views[id(p)] = view
                p.grad = view
                off += p.numel()
                self._index[id(p)] = gi
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))
            self.buckets.append(flat)
            self._seen.append(set())
            self._launched.append(False)
        self._defer = bool(defer_to_scan_end) and self.world > 1
        if self._defer:
            ops.add_scan_backward_listener(self._after_scan_backward)
        if self.world > 1 and on_gpu and dynamic_gemm_order:
            from . import _lib
            if _lib.get_option("gemm_dynamic") < 0:      # an explicit setting wins
                _lib.set_option("gemm_dynamic", 1)

    # ------------------------------------------------------------------ per step
    def zero_grad(self):
        """Zeroes the buckets in place and binds every ``p.grad`` to its slice again."""
        for gi, flat in enumerate(self.buckets):
            flat.zero_()
            for p in self.groups[gi]:
                if p.grad is not self._views[id(p)]:
                    p.grad = self._views[id(p)]
        self._rearm()

    def _rearm(self):
        for gi in range(len(self.buckets)):
            self._seen[gi].clear()
            self._launched[gi] = False
        self._ready = []
        self._handles = []

    def _on_grad(self, p: torch.Tensor):
        gi = self._index[id(p)]
        if self._launched[gi] or id(p) in self._seen[gi]:
            raise RuntimeError(
                "LayerGradAllReducer: a parameter received a second gradient before finish(); run one "
                "backward() per step and call finish() after it")
        view = self._views[id(p)]
        g = p.grad
        if g is not view and not (g is not None and g.data_ptr() == view.data_ptr() and g.dtype == view.dtype
                                  and g.shape == view.shape and g.is_contiguous()):
            # the gradient was detached from its bucket (zero_grad(set_to_none=True), an optimizer that
            # replaced it): this step's value is in the fresh tensor; put it into the bucket and re-bind
            with torch.no_grad():
                view.copy_(g)
            p.grad = view
        self._seen[gi].add(id(p))
        if len(self._seen[gi]) == len(self.groups[gi]):
            if self._defer:
                self._ready.append(gi)
            else:
                self._launch(gi)

    def _after_scan_backward(self):
        """Called right after a backward scan has been enqueued: the buckets completed before it start now."""
        ready, self._ready = self._ready, []
        for gi in ready:
            self._launch(gi)

    def _launch(self, gi: int):
        if self._launched[gi]:
            return
        self._launched[gi] = True
        if self.world <= 1:
            return
        flat = self.buckets[gi]
        if self.reduce_dtype is not None and self.reduce_dtype != flat.dtype:
            wire = flat.to(self.reduce_dtype)
            h = dist.all_reduce(wire, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            self._handles.append((h, gi, wire))
        else:
            h = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            self._handles.append((h, gi, None))

    def finish(self):
        """Starts what backward left (in bucket order, the same on every rank), waits for every all-reduce
        (stream-ordered for NCCL) and re-arms the reducer for the next step."""
        for gi in self._ready:
            self._launch(gi)
        self._ready = []
        for gi in range(len(self.buckets)):
            if not self._launched[gi]:
                # a parameter of this layer got no gradient this step: its slice holds what zero_grad left
                for p in self.groups[gi]:
                    if id(p) not in self._seen[gi] and p.grad is not self._views[id(p)]:
                        if p.grad is not None:
                            with torch.no_grad():
                                self._views[id(p)].copy_(p.grad)
                        p.grad = self._views[id(p)]
                self._launch(gi)
        for h, gi, wire in self._handles:
            h.wait()
            if wire is not None:
                self.buckets[gi].copy_(wire)
        self._rearm()

    # ------------------------------------------------------------------ misc
    def bytes_per_step(self) -> int:
        """Bytes handed to the collective per step."""
        total = 0
        for b in self.buckets:
            size = b.element_size()
            if self.reduce_dtype is not None:
                size = torch.empty((), dtype=self.reduce_dtype).element_size()
            total += b.numel() * size
        return total

    def remove(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []
        if self._defer:
            ops.remove_scan_backward_listener(self._after_scan_backward)
            self._defer = False
