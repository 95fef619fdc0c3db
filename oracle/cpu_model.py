"""CPU execution of the SRU layer stack with the oracle scan.  TEST INFRASTRUCTURE ONLY.

Reuses the package's host-side module classes for parameters and layer plumbing, and
replaces the device operations with CPU ones: the projection becomes ``Tensor.mm``, the layer
normalisation and the recurrence become the C oracle (after the casts of sru/ops.py:116-127, i.e. the
recurrence always runs in float32 unless the tensors are float64).  This is the CPU
baseline that the benchmark times and the model-level checker of the GPU tests.
"""
import copy

import torch

from sru_b200.modules import SRU, SRUCell

from . import sru_oracle


class OracleSRUCell(SRUCell):
    def _apply_recurrence_eager(self, U, V, residual, c0, scale_val, mask_c, mask_pad):
        dt = torch.float64 if U.dtype == torch.float64 else torch.float32
        h, c = sru_oracle.elementwise_recurrence_oracle(
            U.to(dt), residual.to(dt), V.to(dt), self.bias.to(dt), c0.to(dt), self.activation_type,
            self.hidden_size, self.bidirectional, self.has_skip_term,
            None if scale_val is None else scale_val.to(dt),
            None if mask_c is None else mask_c.to(dt), mask_pad)
        return [h, c]

    def _compute_U_eager(self, x):
        if self.weight_proj is not None:
            return x.mm(self.weight_proj).mm(self.weight)
        return x.mm(self.weight)

    def _layer_norm_eager(self, t, before_projection):
        ln = self.layer_norm
        dt = torch.float64 if t.dtype == torch.float64 else torch.float32
        return sru_oracle.layer_norm_oracle(t.to(dt), ln.weight, ln.bias, ln.eps)

    def _begin_grad_link(self, input, residual):
        self._grad_link = None


class OracleSRU(SRU):
    def _restore_output_dtype(self, h, input):
        return h


def to_oracle(model: SRU) -> SRU:
    """A deep copy of `model` on the CPU whose layers compute with the oracle."""
    m = copy.deepcopy(model).cpu()
    m.__class__ = OracleSRU
    for cell in m.rnn_lst:
        cell.__class__ = OracleSRUCell
    return m
