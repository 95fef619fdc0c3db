"""ctypes access to libsru_b200.so (the C ABI of include/sru_b200.h).

There is no fallback: if the library is missing or fails to load, every operator raises.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libsru_b200.so")
TORCH_LIB_PATH = os.path.join(_HERE, "lib", "libsru_b200_torch.so")

SRU_F32, SRU_F16, SRU_BF16, SRU_F64 = 0, 1, 2, 3
DTYPE_CODE = {torch.float32: SRU_F32, torch.float16: SRU_F16, torch.bfloat16: SRU_BF16,
              torch.float64: SRU_F64}

_lib = None
_torch_ops_loaded = False

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int


class SruB200Error(RuntimeError):
    pass


def lib():
    """The loaded C-ABI library.  Raises if it has not been built (python -m sru_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SruB200Error(
                "libsru_b200.so not found at %s: build it with `python -m sru_b200.build`; "
                "this package has no CPU or PyTorch fallback" % LIB_PATH)
        l = ctypes.CDLL(LIB_PATH)
        l.sru_b200_version.restype = _int
        l.sru_b200_last_error.restype = ctypes.c_char_p
        l.sru_b200_check_device_error.restype = _int
        l.sru_b200_check_device_error.argtypes = [_vp]
        l.sru_b200_set_option.restype = _int
        l.sru_b200_set_option.argtypes = [ctypes.c_char_p, _int]
        l.sru_b200_get_option.restype = _int
        l.sru_b200_get_option.argtypes = [ctypes.c_char_p]
        l.sru_b200_last_scan_kernel.restype = _int
        l.sru_b200_last_scan_kernel.argtypes = []
        l.sru_b200_scan_forward.restype = _int
        l.sru_b200_scan_forward.argtypes = [_vp] * 10 + [_i64, _i64, _i64, _int, _int, _int, _int, _int,
                                                         ctypes.c_double, _int, _int, _vp]
        l.sru_b200_scan_backward_workspace_bytes.restype = ctypes.c_size_t
        l.sru_b200_scan_backward_workspace_bytes.argtypes = [_i64, _i64, _i64, _int, _int, _int]
        l.sru_b200_scan_backward.restype = _int
        l.sru_b200_scan_backward.argtypes = [_vp] * 15 + [_i64, _i64, _i64, _int, _int, _int, _int, _int,
                                                          ctypes.c_double, _int, _int, _vp, ctypes.c_size_t, _vp]
        l.sru_b200_gemm.restype = _int
        l.sru_b200_gemm.argtypes = [_vp] * 4 + [_i64] * 6 + [_int] * 5 + [_vp]
        l.sru_b200_gate_bias_columns.restype = _int
        l.sru_b200_gate_bias_columns.argtypes = [_vp, _vp, _i64, _int, _vp]
        l.sru_b200_convert.restype = _int
        l.sru_b200_convert.argtypes = [_vp, _vp, _i64, _int, _int, _vp]
        l.sru_b200_gemm_workspace_bytes.restype = ctypes.c_size_t
        l.sru_b200_gemm_workspace_bytes.argtypes = [_i64, _i64, _i64, _int]
        l.sru_b200_gemm_ws.restype = _int
        l.sru_b200_gemm_ws.argtypes = [_vp] * 4 + [_i64] * 6 + [_int] * 5 + [_vp, ctypes.c_size_t, _vp]
        l.sru_b200_gemm_f32_workspace_bytes.restype = ctypes.c_size_t
        l.sru_b200_gemm_f32_workspace_bytes.argtypes = [_i64, _i64, _i64]
        l.sru_b200_gemm_f32.restype = _int
        l.sru_b200_gemm_f32.argtypes = [_vp] * 4 + [_i64] * 6 + [_int] * 3 + [_vp, ctypes.c_size_t, _vp]
        l.sru_b200_layer_norm_forward.restype = _int
        l.sru_b200_layer_norm_forward.argtypes = [_vp] * 6 + [_i64, _i64, ctypes.c_double, _int, _int, _vp]
        l.sru_b200_layer_norm_backward_workspace_bytes.restype = ctypes.c_size_t
        l.sru_b200_layer_norm_backward_workspace_bytes.argtypes = [_i64, _i64]
        l.sru_b200_layer_norm_backward.restype = _int
        l.sru_b200_layer_norm_backward.argtypes = [_vp] * 8 + [_i64, _i64, _int, _int, _vp, ctypes.c_size_t, _vp]
        _lib = l
    return _lib


def load_torch_ops():
    """Registers torch.ops.sru_cuda.* (the reference's operator names) from the binding library."""
    global _torch_ops_loaded
    if not _torch_ops_loaded:
        if not os.path.exists(TORCH_LIB_PATH):
            raise SruB200Error("libsru_b200_torch.so not found at %s: run `python -m sru_b200.build`"
                               % TORCH_LIB_PATH)
        lib()
        torch.ops.load_library(TORCH_LIB_PATH)
        _torch_ops_loaded = True


SCAN_KERNEL_NAMES = {0: "none", 1: "pipelined", 2: "generic", 3: "split"}


def set_option(name: str, value: int) -> None:
    """Sets a tuning option of the native library (see include/sru_b200.h); negative un-sets it."""
    check(lib().sru_b200_set_option(name.encode(), int(value)))


def get_option(name: str) -> int:
    return int(lib().sru_b200_get_option(name.encode()))


class options:
    """Context manager: ``with options(fwd_v=2, scan_stages=3): ...`` sets, then restores."""

    def __init__(self, **kw):
        self.kw = {k: v for k, v in kw.items() if v is not None}

    def __enter__(self):
        self.old = {k: get_option(k) for k in self.kw}
        for k, v in self.kw.items():
            set_option(k, v)
        return self

    def __exit__(self, *exc):
        for k, v in self.old.items():
            set_option(k, v)


def last_scan_kernel() -> str:
    """'pipelined', 'generic', 'split' or 'none': what this thread's last scan call launched."""
    return SCAN_KERNEL_NAMES.get(int(lib().sru_b200_last_scan_kernel()), "unknown")


def check(rc):
    if rc != 0:
        msg = lib().sru_b200_last_error().decode("utf-8", "replace")
        raise SruB200Error("sru_b200 call failed (%d): %s" % (rc, msg))


def ptr(t):
    return None if t is None else t.data_ptr()


def current_stream_ptr(device=None):
    return torch.cuda.current_stream(device).cuda_stream


def check_device_error(device=None):
    check(lib().sru_b200_check_device_error(current_stream_ptr(device)))


class KernelTimer:
    """Optional per-call timing with CUDA events on the launching stream (used by bench.py).

    Install with ``_lib.timer = KernelTimer()``; every C-ABI launch made through ``call`` is then
    bracketed by a pair of events recorded on the current stream.  ``summary()`` synchronises
    and returns ``{name: (calls, total_ms)}``.
    """

    def __init__(self):
        self.spans = {}

    def add(self, name, start, end):
        self.spans.setdefault(name, []).append((start, end))

    def summary(self):
        torch.cuda.synchronize()
        return {k: (len(v), sum(s.elapsed_time(e) for s, e in v)) for k, v in self.spans.items()}


timer = None          # a KernelTimer, or None
launch_count = 0      # kernels of this library launched so far (bench.py reports the per-step figure)
nvtx_ranges = os.environ.get("SRU_B200_NVTX", "0") not in ("", "0")   # see set_nvtx_ranges


def set_nvtx_ranges(enabled: bool) -> None:
    """Brackets every C-ABI launch with an NVTX range named after its kernel class ("scan_fwd", "gemm_wgrad", ...),
    so that a profiler can filter or group by it (for instance ``ncu --nvtx --nvtx-include "scan_bwd/"``).
    Off by default; also switched on by the environment variable SRU_B200_NVTX=1."""
    global nvtx_ranges
    nvtx_ranges = bool(enabled)


def call(name, n_kernels, fn, *args):
    """Invoke a C-ABI entry point, count its kernel launches, time it if a timer is installed."""
    global launch_count
    launch_count += n_kernels
    if nvtx_ranges:
        torch.cuda.nvtx.range_push(name)
        try:
            return _call(name, fn, *args)
        finally:
            torch.cuda.nvtx.range_pop()
    return _call(name, fn, *args)


def _call(name, fn, *args):
    if timer is None:
        return check(fn(*args))
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    rc = fn(*args)
    end.record()
    timer.add(name, start, end)
    return check(rc)
