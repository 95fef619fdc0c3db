"""Host-to-device input pipeline: the next batch is copied while the current one is being computed.

The reference leaves input transfer to its applications (``x.cuda()`` at the top of each training iteration,
e.g. language_model/train_lm.py); with the recurrence and the projection on B200 kernels a step of the smaller
configurations is as short as the PCIe copy of its input, so that copy is taken off the compute stream.
"""
from typing import Iterable, Iterator, Optional, Sequence, Tuple

import torch
from torch import Tensor


class DevicePrefetcher:
    """Iterates over batches (tuples of pinned host tensors or None), yielding them on ``device``.

    Batch i + 1 is copied on a side stream while the consumer works on batch i.  Two sets of device buffers are used
    in turn (no allocation per step): the consumer's stream waits for a copy's event before the first use of a set, and
    the copy stream waits, before it overwrites a set, for an event recorded on the consumer's stream when the
    consumer asked for the following batch (all its work on the set has been enqueued by then).  A yielded batch is
    therefore valid until the next one is requested: work enqueued on it before that is safe, tensors kept beyond it are
    overwritten.

    >>> for x, mask in DevicePrefetcher(loader, device):     # loader yields (x_pinned, mask_pinned)
    ...     loss = step(x, mask)
    """

    def __init__(self, batches: Iterable[Sequence[Optional[Tensor]]], device):
        self.batches = batches
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("DevicePrefetcher copies to a CUDA device")
        self.stream = torch.cuda.Stream(self.device)
        self._sets = [None, None]          # device tensors of each set
        self._released = [None, None]      # event on the consumer's stream: the set may be overwritten
        # events are re-recorded every step (a wait enqueued earlier keeps the state it saw): no allocation per step
        self._done_ev = [torch.cuda.Event(), torch.cuda.Event()]
        self._rel_ev = [torch.cuda.Event(), torch.cuda.Event()]

    def _start(self, batch, slot: int):
        cur = self._sets[slot]
        if cur is None or len(cur) != len(batch) or any(
                (t is None) != (d is None) or (t is not None and (t.shape != d.shape or t.dtype != d.dtype))
                for t, d in zip(batch, cur)):
            cur = tuple(None if t is None else torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in batch)
            self._sets[slot] = cur
            self._released[slot] = None
        with torch.cuda.stream(self.stream):
            if self._released[slot] is not None:
                self.stream.wait_event(self._released[slot])
            else:
                self.stream.wait_stream(torch.cuda.current_stream(self.device))   # fresh buffers: after their allocation
            for t, d in zip(batch, cur):
                if t is not None:
                    d.copy_(t, non_blocking=True)
            done = self._done_ev[slot]
            done.record(self.stream)
        return cur, done

    def __iter__(self) -> Iterator[Tuple[Optional[Tensor], ...]]:
        pending = None
        slot = 0
        for batch in self.batches:
            started = self._start(batch, slot)
            if pending is not None:
                dev, done = pending
                torch.cuda.current_stream(self.device).wait_event(done)
                yield dev
                # the consumer is back for the next batch: everything it does with `dev` has been enqueued
                rel = self._rel_ev[1 - slot]
                rel.record(torch.cuda.current_stream(self.device))
                self._released[1 - slot] = rel
            pending = started
            slot = 1 - slot
        if pending is not None:
            dev, done = pending
            torch.cuda.current_stream(self.device).wait_event(done)
            yield dev
