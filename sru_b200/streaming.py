"""A sequence that arrives in chunks: the recurrence state is handed from chunk to chunk.

The reference's applications do this by hand for truncated back-propagation and for incremental inference
(language_model/train_enwik8.py:183-193 carries ``hidden`` from one segment to the next).  The final state
the scan returns is float32 whatever the storage type, so a unidirectional stack processed in chunks computes
what one pass over the whole sequence computes -- bit for bit as long as every chunk's projection runs on the same
GEMM as the whole sequence's would (length x batch of each chunk a multiple of 8 for the tensor-core kernel).
"""
from typing import Optional

import torch
from torch import Tensor


class StreamingSRU:
    """Incremental inference over an ``SRU``: ``step(chunk)`` returns the outputs of the chunk and keeps the state.

    >>> stream = StreamingSRU(model.eval())
    >>> for chunk in chunks:                  # each (length_i, batch, input_size)
    ...     h = stream.step(chunk)            # (length_i, batch, output_size)
    >>> stream.reset()                        # before the next, unrelated sequence

    Under ``torch.no_grad()``; every step of a plain stack is one native call (``sru_b200::stack_forward``).
    """

    def __init__(self, model):
        if getattr(model, "bidirectional", False):
            raise ValueError("a bidirectional SRU reads the whole sequence backwards: it cannot be streamed")
        if getattr(model, "nn_rnn_compatible_return", False):
            raise ValueError("streaming keeps the state in the module's own (layers, batch, width) layout; "
                             "construct the SRU with nn_rnn_compatible_return=False")
        self.model = model
        self.state: Optional[Tensor] = None

    def reset(self, state: Optional[Tensor] = None) -> None:
        """Forget the carried state (or start from ``state``: (num_layers, batch, output_size))."""
        self.state = state

    @torch.no_grad()
    def step(self, chunk: Tensor, mask_pad: Optional[Tensor] = None) -> Tensor:
        h, c = self.model(chunk, self.state, mask_pad=mask_pad)
        self.state = c
        return h
