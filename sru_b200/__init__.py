"""B200-native (sm_100a) implementation of the SRU hot path: projection GEMM + light-recurrence scan.

Drop-in for the corresponding part of asappresearch/sru: ``SRU`` / ``SRUCell`` keep the
reference's constructor arguments, call signature and ``state_dict`` layout; the operator
``elementwise_recurrence_gpu`` keeps its signature.  All device work goes through the C ABI
of ``include/sru_b200.h`` (``sru_b200/lib/libsru_b200.so``); there is no CPU or PyTorch fallback.
"""
from . import _lib
from .ops import (ElementwiseRecurrence, elementwise_recurrence_forward, elementwise_recurrence_gpu,
                  get_amp_mode, set_amp_mode, set_c_hist_dtype)

__version__ = "0.1.0"
__all__ = ["ElementwiseRecurrence", "elementwise_recurrence_forward", "elementwise_recurrence_gpu",
           "set_amp_mode", "get_amp_mode", "set_c_hist_dtype"]
