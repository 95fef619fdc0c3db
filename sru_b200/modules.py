"""Host-side mirror of the reference's module API for the hot path: ``SRUCell`` and ``SRU``.

Constructor arguments, ``forward`` signatures, parameter / buffer names and shapes
(``state_dict`` layout) and the initialisation recipe are those of sru/modules.py
(``SRUCell`` :16-420, ``SRU`` :422-689), so a checkpoint of the reference loads unchanged
and a model built under the same RNG seed has the same weights.  What differs is below the
operator boundary: ``compute_U`` (sru/modules.py:363-378) runs on the tcgen05 GEMM of this
package for 16-bit operands, and ``apply_recurrence`` (sru/modules.py:283-318) calls the
sm_100a scan kernels.  CUDA only: there is no CPU execution path.
"""
import copy
import math
import warnings
from typing import List, Optional, Tuple, Union

import torch
import torch.nn as nn
from torch import Tensor
from torch.nn.utils.rnn import PackedSequence

from . import _lib
from . import ops
from .layer_norm import layer_norm
from .projection import (GradLink, bias_fold_enabled, gate_bias_columns, gemm_backend, grad_link_enabled,
                         project, will_run_native)


def _load_scripted_ops() -> bool:
    try:
        _lib.load_torch_ops()
        return True
    except Exception:  # binding not built: eager mode still works, scripting raises
        return False


_HAVE_TORCH_OPS = _load_scripted_ops()
_native_stack_enabled = True


def set_native_stack_enabled(enabled: bool) -> None:
    """Whether an inference ``SRU.forward`` of plain layers runs its layer loop as one native call
    (``sru_b200::stack_forward``; default) or as the Python loop over ``SRUCell.forward_native``."""
    global _native_stack_enabled
    _native_stack_enabled = bool(enabled)

if _HAVE_TORCH_OPS:

    @torch.jit.script
    def elementwise_recurrence_inference(U: Tensor, x: Tensor, weight_c: Tensor, bias: Tensor,
                                         c_init: Tensor, activation_type: int, hidden_size: int,
                                         bidirectional: bool, has_skip_term: bool,
                                         scale_x: Optional[Tensor] = None,
                                         dropout_mask_c: Optional[Tensor] = None,
                                         mask_pad: Optional[Tensor] = None) -> List[Tensor]:
        """TorchScript path (sru/ops.py:22-94, sru/cuda_functional.py:37-153): reaches the
        kernels through the registered ``sru_cuda::*`` operators.  CUDA tensors only."""
        assert dropout_mask_c is None, "Dropout mask cannot be set during inference"
        assert U.is_cuda, "sru_b200 has no CPU path"
        d = hidden_size
        length = x.size(0) if x.dim() == 3 else 1
        batch = x.size(-2)
        k = U.size(-1) // d
        k_ = k // 2 if bidirectional else k
        is_custom = 1 if weight_c.dim() > 1 else 0
        skip_type = 0
        if has_skip_term:
            skip_type = 1 if k_ == 3 else 2
        pad: Optional[Tensor] = None
        if mask_pad is not None:
            pad = mask_pad.to(dtype=torch.bool).contiguous()
        x_: Optional[Tensor] = None
        if skip_type == 1:
            x_ = x.contiguous() * scale_x if scale_x is not None else x.contiguous()
        simple = (k_ == 3) and has_skip_term and (is_custom == 0) and (activation_type == 0)
        if simple and bidirectional:
            h, c = torch.ops.sru_cuda.sru_bi_forward_simple(
                U.contiguous(), x_, weight_c.contiguous(), bias, c_init.contiguous(), None, pad,
                length, batch, d)
        elif simple:
            h, c = torch.ops.sru_cuda.sru_forward_simple(
                U.contiguous(), x_, weight_c.contiguous(), bias, c_init.contiguous(), None, pad,
                length, batch, d)
        elif bidirectional:
            h, c = torch.ops.sru_cuda.sru_bi_forward(
                U.contiguous(), x_, weight_c.contiguous(), bias, c_init.contiguous(), None, pad,
                length, batch, d, k_, activation_type, skip_type, is_custom)
        else:
            h, c = torch.ops.sru_cuda.sru_forward(
                U.contiguous(), x_, weight_c.contiguous(), bias, c_init.contiguous(), None, pad,
                length, batch, d, k_, activation_type, skip_type, is_custom)
        if x.dim() == 2:
            return [h.squeeze(0), c.squeeze(0)]
        if bidirectional:
            return [h, torch.cat((c[-1, :, :d], c[0, :, d:]), dim=1)]
        return [h, c[-1]]

else:

    @torch.jit.unused
    def elementwise_recurrence_inference(U: Tensor, x: Tensor, weight_c: Tensor, bias: Tensor,
                                         c_init: Tensor, activation_type: int, hidden_size: int,
                                         bidirectional: bool, has_skip_term: bool,
                                         scale_x: Optional[Tensor] = None,
                                         dropout_mask_c: Optional[Tensor] = None,
                                         mask_pad: Optional[Tensor] = None) -> List[Tensor]:
        raise _lib.SruB200Error("TorchScript needs libsru_b200_torch.so: run `python -m sru_b200.build`")


class SRUCell(nn.Module):
    """One SRU layer.  Same arguments as the reference's ``SRUCell`` (sru/modules.py:30-46)."""

    __constants__ = ['input_size', 'hidden_size', 'output_size', 'rnn_dropout', 'dropout',
                     'bidirectional', 'has_skip_term', 'highway_bias', 'v1', 'rescale',
                     'activation_type', 'activation', 'custom_m', 'projection_size', 'num_matrices',
                     'layer_norm', 'weight_proj', 'scale_x', 'normalize_after', 'weight_c_init']

    scale_x: Tensor
    weight_proj: Optional[Tensor]

    def __init__(self, input_size: int, hidden_size: int, dropout: float = 0.0, rnn_dropout: float = 0.0,
                 bidirectional: bool = False, n_proj: int = 0, use_tanh: bool = False,
                 highway_bias: float = 0.0, has_skip_term: bool = True, layer_norm: bool = False,
                 rescale: bool = True, v1: bool = False, custom_m: Optional[nn.Module] = None,
                 amp_recurrence_fp16: bool = False, normalize_after: bool = False,
                 weight_c_init: Optional[float] = None):
        super().__init__()
        dirs = 2 if bidirectional else 1
        self.input_size = input_size
        self.hidden_size = hidden_size            # per direction
        self.output_size = hidden_size * dirs
        self.rnn_dropout = float(rnn_dropout)
        self.dropout = float(dropout)
        self.bidirectional = bidirectional
        self.has_skip_term = has_skip_term
        self.highway_bias = highway_bias
        self.v1 = v1
        self.rescale = rescale
        self.activation_type = 1 if use_tanh else 0
        self.activation = 'tanh' if use_tanh else 'none'
        self.custom_m: Optional[nn.Module] = custom_m
        self.amp_recurrence_fp16 = amp_recurrence_fp16
        self.normalize_after = normalize_after
        self.weight_c_init = weight_c_init

        # low-rank factor only when it is actually narrower than both sides
        self.projection_size = n_proj if 0 < n_proj < min(self.input_size, self.output_size) else 0
        # a fourth gate column carries the highway input when it cannot be x itself
        self.num_matrices = 4 if (has_skip_term and self.input_size != self.output_size) else 3

        n_cols = self.output_size * self.num_matrices
        if self.custom_m is None:
            if self.projection_size == 0:
                self.weight_proj = None
                self.weight = nn.Parameter(torch.Tensor(input_size, n_cols))
            else:
                self.weight_proj = nn.Parameter(torch.Tensor(input_size, self.projection_size))
                self.weight = nn.Parameter(torch.Tensor(self.projection_size, n_cols))
        self.weight_c = nn.Parameter(torch.Tensor(2 * self.output_size))
        self.bias = nn.Parameter(torch.Tensor(2 * self.output_size))
        self.register_buffer('scale_x', torch.FloatTensor([0]))

        self.layer_norm: Optional[nn.Module] = None
        if layer_norm:
            self.layer_norm = nn.LayerNorm(self.output_size if normalize_after else self.input_size)
        self.reset_parameters()

    def reset_parameters(self):
        """Initialisation recipe of sru/modules.py:164-233 (same order of random draws)."""
        D = self.output_size
        hb = self.highway_bias
        highway_scale = (1.0 + 2.0 * math.exp(hb)) ** 0.5
        with torch.no_grad():
            self.bias.zero_()
            self.bias[D:].fill_(hb)
            self.scale_x[0] = highway_scale if (self.rescale and self.has_skip_term) else 1.0
            ops.forget_scale(self.scale_x)
            self.__dict__.pop("_inference_operands", None)

            gates = None
            if self.custom_m is None:
                fan_in = self.weight.size(0)
                bound = (3.0 / fan_in) ** 0.5
                self.weight.uniform_(-bound, bound)
                if self.projection_size > 0:
                    bound = (3.0 / self.weight_proj.size(0)) ** 0.5
                    self.weight_proj.uniform_(-bound, bound)
                # (fan_in, directions, hidden, gate): the gate index is innermost in memory
                gates = self.weight.view(fan_in, -1, self.hidden_size, self.num_matrices)
                if self.dropout > 0:
                    gates[..., 0].mul_((1 - self.dropout) ** 0.5)
                if self.rnn_dropout > 0:
                    gates.mul_((1 - self.rnn_dropout) ** 0.5)
                if self.layer_norm:
                    gates.mul_(0.1)
                if self.rescale and self.has_skip_term and self.num_matrices == 4:
                    gates[..., 3].mul_(highway_scale)
            elif hasattr(self.custom_m, 'reset_parameters'):
                self.custom_m.reset_parameters()
            else:
                warnings.warn("Unable to reset parameters for custom module. reset_parameters() method "
                              "not found for custom module. " + self.custom_m.__class__.__name__)

            if self.v1:
                self.weight_c.zero_()
                self.weight_c.requires_grad = False
            else:
                if self.weight_c_init is None:
                    self.weight_c.uniform_(-3.0 ** 0.5, 3.0 ** 0.5)
                    self.weight_c.mul_(0.5 ** 0.5)
                else:
                    self.weight_c.uniform_(-self.weight_c_init, self.weight_c_init)
                if gates is not None:
                    gates[..., 1].mul_(0.5 ** 0.5)
                    gates[..., 2].mul_(0.5 ** 0.5)

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        ops.forget_scale(self.scale_x)
        self.__dict__.pop("_inference_operands", None)

    def train(self, mode: bool = True):
        self.__dict__.pop("_inference_operands", None)     # copies kept by the native inference loop
        return super().train(mode)

    def _apply(self, fn, *args, **kwargs):
        self.__dict__.pop("_inference_operands", None)     # .to() / .cuda() / .half() replace the parameters
        return super()._apply(fn, *args, **kwargs)

    def forward(self, input: Tensor, c0: Optional[Tensor] = None,
                mask_pad: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        """(length, batch, input_size) or (batch, input_size) -> (h, c_last), as sru/modules.py:235-281.
        A layer called on its own hands back the types the reference would (float32 h for float32 input under
        16-bit autocast); inside an ``SRU`` stack the layers pass the 16-bit h on (``forward_native``)."""
        h, c = self.forward_native(input, c0, mask_pad)
        if not torch.jit.is_scripting():
            h = self._restore_output_dtype(h, input)
        return h, c

    @torch.jit.unused
    def _restore_output_dtype(self, h: Tensor, input: Tensor) -> Tensor:
        if ops.get_amp_mode() == "native" and h.dtype in (torch.float16, torch.bfloat16) \
                and input.dtype == torch.float32 and not self.amp_recurrence_fp16:
            return ops.widen_to_float32(h)
        return h

    def forward_native(self, input: Tensor, c0: Optional[Tensor] = None,
                       mask_pad: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        """The layer, with h left in the type the recurrence wrote it in."""
        if input.dim() != 2 and input.dim() != 3:
            raise ValueError("Input must be 2 or 3 dimensional")
        batch_size = input.size(-2)
        if c0 is None:
            c0 = torch.zeros(batch_size, self.output_size, dtype=input.dtype, device=input.device)

        residual = input
        if self.layer_norm is not None and not self.normalize_after:
            if not torch.jit.is_scripting():
                input = self._layer_norm_eager(input, True)
            else:
                input = self._layer_norm_scripted(input)
        if self.training and (self.rnn_dropout > 0):
            mask = self.get_dropout_mask_((batch_size, input.size(-1)), self.rnn_dropout)
            input = input * mask.expand_as(input)

        scale_val: Optional[Tensor] = None
        scale_val = self.scale_x if self.rescale else None
        mask_c: Optional[Tensor] = None
        if self.training and (self.dropout > 0):
            if not torch.jit.is_scripting():
                mask_c = self._take_preset_mask(batch_size)
            if mask_c is None:
                mask_c = self.get_dropout_mask_((batch_size, self.output_size), self.dropout)

        if not torch.jit.is_scripting():
            self._begin_grad_link(input, residual)
        U, V = self.compute_UV(input, c0, mask_pad)
        h, c = self.apply_recurrence(U, V, residual, c0, scale_val, mask_c, mask_pad)
        if self.layer_norm is not None and self.normalize_after:
            if not torch.jit.is_scripting():
                h = self._layer_norm_eager(h, False)
            else:
                h = self._layer_norm_scripted(h)
        return h, c

    def _layer_norm_scripted(self, t: Tensor) -> Tensor:
        """The layer's nn.LayerNorm on this package's kernel, for the scripted (inference) path."""
        ln = self.layer_norm
        assert ln is not None
        return torch.ops.sru_b200.layer_norm(t, ln.weight, ln.bias, ln.eps)

    @torch.jit.unused
    def _layer_norm_eager(self, t: Tensor, before_projection: bool) -> Tensor:
        """The layer's nn.LayerNorm (sru/modules.py:252-253, :278-279) on this package's kernel.

        Output type: before the projection, inside a 16-bit autocast region with the tcgen05 GEMM
        and no input dropout, the normalised rows are written in the autocast type (they only feed the
        GEMM, which would round them to that type anyway).  After the recurrence, native amp mode keeps
        a 16-bit h in its type.  Otherwise the reference's types: float32 under autocast, else t's.
        """
        ln = self.layer_norm
        out_dtype: Optional[torch.dtype] = None
        if before_projection:
            if (torch.is_autocast_enabled("cuda") and gemm_backend() == "tcgen05" and self.custom_m is None
                    and not (self.training and self.rnn_dropout > 0)):
                out_dtype = torch.get_autocast_dtype("cuda")
        elif ops.get_amp_mode() == "native" and t.dtype in (torch.float16, torch.bfloat16):
            out_dtype = t.dtype
        return layer_norm(t, ln.weight, ln.bias, ln.eps, out_dtype)

    def apply_recurrence(self, U: Tensor, V: Tensor, residual: Tensor, c0: Tensor,
                         scale_val: Optional[Tensor], mask_c: Optional[Tensor],
                         mask_pad: Optional[Tensor]) -> List[Tensor]:
        if not torch.jit.is_scripting():
            return self._apply_recurrence_eager(U, V, residual, c0, scale_val, mask_c, mask_pad)
        else:
            return elementwise_recurrence_inference(U, residual, V, self.bias, c0, self.activation_type,
                                                    self.hidden_size, self.bidirectional,
                                                    self.has_skip_term, scale_val, mask_c, mask_pad)

    @torch.jit.unused
    def _begin_grad_link(self, input: Tensor, residual: Tensor) -> None:
        """A k = 3 layer whose GEMM operand and highway input are one tensor gets a GradLink: the two
        gradients of that tensor are then summed in the dgrad GEMM's epilogue instead of by autograd."""
        self._grad_link = None
        if (grad_link_enabled() and input is residual and self.custom_m is None and self.weight_proj is None
                and self.has_skip_term and self.num_matrices == 3 and input.is_cuda
                and torch.is_grad_enabled() and input.requires_grad):
            self._grad_link = GradLink()

    @torch.jit.unused
    def _apply_recurrence_eager(self, U: Tensor, V: Tensor, residual: Tensor, c0: Tensor,
                                scale_val: Optional[Tensor], mask_c: Optional[Tensor],
                                mask_pad: Optional[Tensor]) -> List[Tensor]:
        link, self._grad_link = getattr(self, "_grad_link", None), None
        folded, self._bias_folded = getattr(self, "_bias_folded", False), False
        return ops.elementwise_recurrence_gpu(U, residual, V, self.bias, c0, self.activation_type,
                                              self.hidden_size, self.bidirectional, self.has_skip_term,
                                              scale_val, mask_c, mask_pad, self.amp_recurrence_fp16,
                                              grad_link=link, bias_in_u=folded)

    def compute_UV(self, input: Tensor, c0: Optional[Tensor],
                   mask_pad: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
        """U (and the optional per-step V of a custom module), as sru/modules.py:321-361."""
        if self.custom_m is None:
            return self.compute_U(input), self.weight_c
        ret = self.custom_m(input)
        if isinstance(ret, (tuple, list)):
            if len(ret) > 2:
                raise Exception("Custom module must return 1 or 2 tensors but got {}.".format(len(ret)))
            U, V = ret[0], ret[1] + self.weight_c
        else:
            U, V = ret, self.weight_c
        if U.size(-1) != self.output_size * self.num_matrices:
            raise ValueError("U must have a last dimension of {} but got {}.".format(
                self.output_size * self.num_matrices, U.size(-1)))
        if V.size(-1) != self.output_size * 2:
            raise ValueError("V must have a last dimension of {} but got {}.".format(
                self.output_size * 2, V.size(-1)))
        return U, V

    def compute_U(self, input: Tensor) -> Tensor:
        """U = x W (through W_proj first when factorised): (length*batch, output_size*num_matrices)."""
        x = input if input.dim() == 2 else input.contiguous().view(-1, self.input_size)
        if not torch.jit.is_scripting():
            return self._compute_U_eager(x)
        # scripted (inference) path: this package's GEMM through its registered operator; the operator itself
        # hands operands it does not take (fp32, unaligned shapes) to the library product
        weight_proj = self.weight_proj
        if weight_proj is not None:
            x = torch.ops.sru_b200.gemm(x, weight_proj, None)
        return torch.ops.sru_b200.gemm(x, self.weight, None)

    @torch.jit.unused
    def _compute_U_eager(self, x: Tensor) -> Tensor:
        """The projection on this package's GEMM.  When that GEMM is the tcgen05 kernel (16-bit compute type), the
        gate bias is added to U in its epilogue and the recurrence is told so (it then runs without a bias and still
        returns grad_bias); other products leave the bias to the recurrence, as the reference does."""
        self._bias_folded = False
        if self.weight_proj is not None:
            x = project(x, self.weight_proj)
        col_bias = None
        if bias_fold_enabled() and will_run_native(x, self.weight):
            col_bias = gate_bias_columns(self.bias, self.output_size, self.num_matrices)
            self._bias_folded = True
        link = getattr(self, "_grad_link", None) if self.weight_proj is None else None
        return project(x, self.weight, col_bias=col_bias, link=link)

    def get_dropout_mask_(self, size: Tuple[int, int], p: float) -> Tensor:
        """Inverted-dropout mask shared over time (sru/modules.py:380-387)."""
        b = self.bias.data
        return b.new_empty(size).bernoulli_(1 - p).div_(1 - p)

    @torch.jit.unused
    def _take_preset_mask(self, batch_size: int) -> Optional[Tensor]:
        """The mask an enclosing ``SRU`` drew for this layer and this call (all layers' masks come from one
        launch there), or None."""
        m = self.__dict__.get("_preset_mask_c")
        if m is None:
            return None
        self.__dict__["_preset_mask_c"] = None
        return m if m.shape == (batch_size, self.output_size) else None

    def extra_repr(self):
        parts = ["{}, {}".format(self.input_size, self.hidden_size)]
        if self.projection_size > 0:
            parts.append("projection_size={}".format(self.projection_size))
        if self.dropout > 0:
            parts.append("dropout={}".format(self.dropout))
        if self.rnn_dropout > 0:
            parts.append("rnn_dropout={}".format(self.rnn_dropout))
        if self.bidirectional:
            parts.append("bidirectional=True")
        if self.highway_bias != 0:
            parts.append("highway_bias={}".format(self.highway_bias))
        if self.activation_type != 0:
            parts.append("activation={}".format(self.activation))
        if self.v1:
            parts.append("v1=True")
        parts.append("rescale={}".format(self.rescale))
        if not self.has_skip_term:
            parts.append("has_skip_term=False")
        if self.layer_norm:
            parts.append("layer_norm=True")
        s = ", ".join(parts)
        if self.custom_m is not None:
            s += ",\n  custom_m=" + str(self.custom_m)
        return s

    def __repr__(self):
        s = self.extra_repr()
        if len(s.split('\n')) == 1:
            return "{}({})".format(self.__class__.__name__, s)
        return "{}({}\n)".format(self.__class__.__name__, s)


class SRU(nn.Module):
    """Stack of SRU layers.  Same arguments as the reference's ``SRU`` (sru/modules.py:432-451)."""

    __constants__ = ['input_size', 'hidden_size', 'output_size', 'num_layers', 'dropout', 'rnn_dropout',
                     'projection_size', 'rnn_lst', 'bidirectional', 'use_layer_norm', 'has_skip_term',
                     'num_directions', 'nn_rnn_compatible_return', 'input_to_hidden']

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 2, dropout: float = 0.0,
                 rnn_dropout: float = 0.0, bidirectional: bool = False, projection_size: int = 0,
                 use_tanh: bool = False, layer_norm: bool = False, highway_bias: float = 0.0,
                 has_skip_term: bool = True, rescale: bool = False, v1: bool = False,
                 nn_rnn_compatible_return: bool = False,
                 custom_m: Optional[Union[nn.Module, List[nn.Module]]] = None,
                 proj_input_to_hidden_first: bool = False, amp_recurrence_fp16: bool = False,
                 normalize_after: bool = False, weight_c_init: Optional[float] = None):
        super().__init__()
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.num_directions = 2 if bidirectional else 1
        self.output_size = hidden_size * self.num_directions
        self.num_layers = num_layers
        self.dropout = dropout
        self.rnn_dropout = rnn_dropout
        self.projection_size = projection_size
        self.bidirectional = bidirectional
        self.use_layer_norm = layer_norm
        self.has_skip_term = has_skip_term
        self.nn_rnn_compatible_return = nn_rnn_compatible_return
        self.amp_recurrence_fp16 = amp_recurrence_fp16
        self.input_to_hidden = None
        first_in = input_size
        if proj_input_to_hidden_first and input_size != self.output_size:
            first_in = self.output_size
            self.input_to_hidden = nn.Linear(input_size, self.output_size, bias=False)

        if rnn_dropout > 0:
            warnings.warn("rnn_dropout > 0 is deprecated and will be removed in"
                          "next major version of SRU. Please use dropout instead.")
        if use_tanh:
            warnings.warn("use_tanh = True is deprecated and will be removed in"
                          "next major version of SRU.")

        layers = nn.ModuleList()
        for i in range(num_layers):
            m_i = None
            if custom_m is not None:
                m_i = custom_m[i] if isinstance(custom_m, list) else copy.deepcopy(custom_m)
            layers.append(SRUCell(
                first_in if i == 0 else self.output_size, hidden_size,
                dropout=dropout if i + 1 != num_layers else 0,   # no dropout after the last layer
                rnn_dropout=rnn_dropout, bidirectional=bidirectional, n_proj=projection_size,
                use_tanh=use_tanh, layer_norm=layer_norm, highway_bias=highway_bias,
                has_skip_term=has_skip_term, rescale=rescale, v1=v1, custom_m=m_i,
                amp_recurrence_fp16=amp_recurrence_fp16, normalize_after=normalize_after,
                weight_c_init=weight_c_init))
        self.rnn_lst = layers

    def forward(self, input: Tensor, c0: Optional[Tensor] = None,
                mask_pad: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        """(length, batch, input_size) [or a PackedSequence] -> (h, stacked last states).

        c0: (num_layers, batch, output_size); mask_pad: (length, batch), non-zero = padding.
        Returns h (length, batch, output_size) and c (num_layers, batch, output_size), or
        (num_layers*num_directions, batch, hidden_size) with ``nn_rnn_compatible_return``
        (sru/modules.py:572-652).
        """
        orig_input = input
        if isinstance(orig_input, PackedSequence):
            input, lengths = nn.utils.rnn.pad_packed_sequence(input)
            steps = torch.arange(int(lengths.max().item())).unsqueeze(1)
            mask_pad = (steps >= lengths.unsqueeze(0)).to(torch.uint8).to(input.device).contiguous()
        if input.dim() != 3:
            raise ValueError("There must be 3 dimensions for (length, batch_size, input_size)")

        if c0 is None:
            zeros = torch.zeros(input.size(1), self.output_size, dtype=input.dtype, device=input.device)
            c0_ = [zeros for _ in range(self.num_layers)]
        else:
            if c0.dim() != 3:
                raise ValueError("c0 must be 3 dim (num_layers, batch_size, output_size)")
            c0_ = [x.squeeze(0) for x in c0.chunk(self.num_layers, 0)]

        prevx = input if self.input_to_hidden is None else self.input_to_hidden(input)
        native: Optional[List[Tensor]] = None
        if not torch.jit.is_scripting():
            native = self._forward_native_stack(prevx, c0, mask_pad)
        if native is not None:
            prevx, lstc_stack = native[0], native[1]
        else:
            if not torch.jit.is_scripting():
                self._preset_dropout_masks(input.size(1))
            lstc = []
            i = 0
            for rnn in self.rnn_lst:
                h, c = rnn.forward_native(prevx, c0_[i], mask_pad=mask_pad)
                prevx = h
                lstc.append(c)
                i += 1
            lstc_stack = torch.stack(lstc)
        if not torch.jit.is_scripting():
            prevx = self._restore_output_dtype(prevx, input)

        if self.nn_rnn_compatible_return:
            batch_size = input.size(1)
            lstc_stack = lstc_stack.view(self.num_layers, batch_size, self.num_directions, self.hidden_size)
            lstc_stack = lstc_stack.transpose(1, 2).contiguous()
            lstc_stack = lstc_stack.view(self.num_layers * self.num_directions, batch_size, self.hidden_size)

        if isinstance(orig_input, PackedSequence):
            prevx = nn.utils.rnn.pack_padded_sequence(prevx, lengths, enforce_sorted=False)
        return prevx, lstc_stack

    @torch.jit.unused
    def _forward_native_stack(self, x: Tensor, c0: Optional[Tensor], mask_pad: Optional[Tensor]) -> Optional[List[Tensor]]:
        """Inference through ``sru_b200::stack_forward``: the whole layer loop as one native call (one Python to
        C++ transition instead of several per layer; same kernels and arguments as the loop, identical results).
        Returns None when the stack or the call is not of the plain kind that operator serves: gradients needed,
        training mode, factorised or custom projections, a non-identity activation, fp32 compute, widths the
        kernels do not take, the per-kernel timer of the benchmark installed."""
        if (not _HAVE_TORCH_OPS or not _native_stack_enabled or torch.is_grad_enabled() or self.training
                or not x.is_cuda or x.dim() != 3 or _lib.timer is not None or ops.get_amp_mode() != "native"
                or gemm_backend() != "tcgen05" or not bias_fold_enabled()):
            return None
        length, batch = x.size(0), x.size(1)
        if length == 0 or (length * batch) % 8 != 0:
            return None
        first = self.rnn_lst[0]
        autocast = torch.is_autocast_enabled("cuda")
        dt = torch.get_autocast_dtype("cuda") if autocast else (
            first.weight.dtype if first.weight.dtype != x.dtype else x.dtype)
        if dt not in (torch.float16, torch.bfloat16):
            return None
        # what the first layer reads: under autocast a float32 input stays float32 for the first layer norm (the
        # module's own path normalises the unrounded rows); everything else enters in the compute type
        if x.dtype not in (torch.float32, dt) or (x.dtype == torch.float32 and not autocast):
            return None
        D = self.output_size
        width = x.size(2)
        ks: List[int] = []
        skips: List[int] = []
        scales: List[float] = []
        has_norm: List[int] = []
        ln_w: List[Tensor] = []
        ln_b: List[Tensor] = []
        ln_eps: List[float] = []
        none = x.new_empty(0)
        w_list: List[Tensor] = []
        cb_list: List[Tensor] = []
        normalize_after = bool(first.normalize_after)
        for cell in self.rnn_lst:
            k = cell.num_matrices
            if (cell.weight_proj is not None or cell.custom_m is not None
                    or cell.activation_type != 0 or cell.amp_recurrence_fp16 or cell.output_size != D
                    or cell.weight.size(0) != width or width % 8 != 0 or (D * k) % 8 != 0
                    or cell.weight.dtype not in (torch.float32, dt) or not cell.weight.is_cuda
                    or bool(cell.normalize_after) != normalize_after):
                return None
            ln = cell.layer_norm
            if ln is not None:
                rows = D if normalize_after else width
                if tuple(ln.normalized_shape) != (rows,) or rows > 4096:
                    return None
                ln_w.append(none if ln.weight is None else ln.weight)
                ln_b.append(none if ln.bias is None else ln.bias)
                ln_eps.append(float(ln.eps))
            else:
                ln_w.append(none)
                ln_b.append(none)
                ln_eps.append(0.0)
            has_norm.append(0 if ln is None else 1)
            # the weight in the compute type and the gate bias laid out over U's columns are kept between calls
            # (inference weights do not change; the key follows in-place updates autograd can see, and
            # reset_parameters / load_state_dict / train() drop the copies)
            try:
                key = (cell.weight.data_ptr(), cell.weight._version, cell.bias.data_ptr(), cell.bias._version, dt)
            except RuntimeError:        # parameters made in inference mode track no version: nothing is kept
                key = None
            kept = cell.__dict__.get("_inference_operands")
            if key is None or kept is None or kept[0] != key:
                w16 = cell.weight.detach() if cell.weight.dtype == dt else cell.weight.detach().to(dt)
                kept = (key, w16.contiguous(), gate_bias_columns(cell.bias.detach(), D, k))
                cell.__dict__["_inference_operands"] = kept
            w_list.append(kept[1])
            cb_list.append(kept[2])
            ks.append(k)
            skips.append(0 if not cell.has_skip_term else (1 if k == 3 else 2))
            scales.append(ops._scale_value(cell.scale_x if cell.rescale else None))
            width = D
        if c0 is not None and (c0.dim() != 3 or c0.size(0) != self.num_layers):
            return None
        out = torch.ops.sru_b200.stack_forward(
            x, w_list, [c.weight_c for c in self.rnn_lst], [c.bias for c in self.rnn_lst],
            scales, c0, mask_pad, self.hidden_size, self.bidirectional, ks, skips, dt == torch.float16,
            has_norm, ln_w, ln_b, ln_eps, normalize_after, cb_list)
        _lib.launch_count += 2 * len(ks) + sum(has_norm)      # per layer: product, scan (+ layer norm)
        return [out[0], out[1]]

    @torch.jit.unused
    def _preset_dropout_masks(self, batch_size: int) -> None:
        """Draws the dropout masks of all layers with ONE bernoulli launch (the reference draws one per layer,
        sru/modules.py:380-387; same distribution, two launches per step instead of two per layer).  Layers whose
        ``get_dropout_mask_`` was replaced on the instance keep drawing their own."""
        if not self.training:
            return
        cells = [c for c in self.rnn_lst if c.dropout > 0 and "get_dropout_mask_" not in c.__dict__]
        if len(cells) < 2:
            return
        first = cells[0]
        if any(c.dropout != first.dropout or c.output_size != first.output_size
               or c.bias.device != first.bias.device or c.bias.dtype != first.bias.dtype for c in cells):
            return
        p = first.dropout
        masks = first.bias.data.new_empty((len(cells), batch_size, first.output_size)).bernoulli_(1 - p).div_(1 - p)
        for i, c in enumerate(cells):
            c.__dict__["_preset_mask_c"] = masks[i]

    @torch.jit.unused
    def _restore_output_dtype(self, h: Tensor, input: Tensor) -> Tensor:
        """In native amp mode layers hand 16-bit h to each other; the caller gets the dtype the
        reference would return (float32 under autocast, see sru/ops.py:116-127)."""
        if ops.get_amp_mode() == "native" and h.dtype in (torch.float16, torch.bfloat16) \
                and input.dtype == torch.float32 and not self.amp_recurrence_fp16:
            return ops.widen_to_float32(h)
        return h

    def reset_parameters(self):
        for rnn in self.rnn_lst:
            rnn.reset_parameters()
        if self.input_to_hidden is not None:
            self.input_to_hidden.reset_parameters()

    def make_backward_compatible(self):
        """Fills in attributes that checkpoints pickled by older releases lack (sru/modules.py:660-689)."""
        self.nn_rnn_compatible_return = getattr(self, 'nn_rnn_compatible_return', False)
        if hasattr(self, 'n_in'):  # releases <= 2.1.7 used other attribute names
            if len(self.ln_lst):
                raise Exception("Layer norm is not backward compatible for sru<=2.1.7")
            if self.use_weight_norm:
                raise Exception("Weight norm removed in sru>=2.1.9")
            self.input_size, self.hidden_size, self.output_size = self.n_in, self.n_out, self.out_size
            self.num_layers, self.projection_size, self.use_layer_norm = self.depth, self.n_proj, False
            for cell in self.rnn_lst:
                cell.input_size, cell.hidden_size = cell.n_in, cell.n_out
                cell.output_size = cell.n_out * 2 if cell.bidirectional else cell.n_out
                cell.num_matrices, cell.projection_size, cell.layer_norm = cell.k, cell.n_proj, None
                if cell.activation_type > 1:
                    raise Exception("ReLU or SeLU activation removed in sru>=2.1.9")
        if not hasattr(self, 'input_to_hidden'):  # releases <= 2.1.9
            self.input_to_hidden = None
            for cell in self.rnn_lst:
                cell.custom_m = None
