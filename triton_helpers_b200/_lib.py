r"""ctypes binding of ``libth_b200.so`` (declared in ``include/th_b200.h``).

The library is the only compute path: there is no Triton, eager-PyTorch or CPU fallback.
If the shared object has not been built, loading raises with the build command; every
non-zero return code of an entry point becomes a ``RuntimeError`` carrying
``th_last_error_string()``.
"""
import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from functools import lru_cache
from pathlib import Path
from typing import Optional, Sequence

import torch
from torch import Tensor

LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libth_b200.so"

DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
ACTIVATION_CODE = {"none": 0, "relu": 1, "silu": 2, "relu2": 3}
TH_ERR_UNSUPPORTED = -2  # include/th_b200.h

_I32P = ctypes.POINTER(c_int32)
_I64P = ctypes.POINTER(c_int64)

# name -> (restype, argtypes); every symbol include/th_b200.h declares
SIGNATURES = {
    "th_version": (c_int, []),
    "th_last_error_string": (c_char_p, []),
    "th_hash_fwd": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int, c_int, c_int,
         _I32P, _I64P, _I64P, _I64P, c_float, c_int, c_int, c_void_p],
    ),
    "th_hash_bwd": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int, c_int64, c_int, c_int, c_int,
         _I32P, _I64P, _I64P, _I64P, c_float, c_int, c_int, c_void_p],
    ),
    "th_hash_debug_indices": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, _I32P, _I64P, _I64P,
         c_float, c_void_p],
    ),
    "th_hash_status": (c_int, []),
    "th_field_fwd": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int, c_void_p, c_int, c_int, c_int, _I32P, _I64P, _I64P, _I64P, c_float,
         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
         c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_float, c_int64, c_int,
         c_void_p],
    ),
    "th_field_workspace_bytes": (c_int64, [c_int, c_int, c_int, c_int, c_int]),
    "th_field_bwd": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, _I32P, _I64P, _I64P, _I64P, c_float,
         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
         c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int, c_void_p],
    ),
    "th_mlp_fwd": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "th_mlp_fwd_mse": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
         c_int64, c_void_p, c_int64, c_void_p, c_float, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "th_mlp_workspace_bytes": (c_int64, [c_int, c_int, c_int, c_int]),
    "th_mlp_tc_status": (c_int, []),
    "th_mlp_tma_available": (c_int, []),
    "th_mlp_bwd": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "th_mlp_bwd_static": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "th_mlp_bwd_static_max_bytes": (c_int64, []),
    "th_rev_fwd": (
        c_int,
        [c_void_p, c_int64] + [c_void_p] * 8 + [c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "th_rev_workspace_bytes": (c_int64, [c_int64, c_int, c_int, c_int]),
    "th_rev_tc_status": (c_int, []),
    "th_rev_bwd": (
        c_int,
        [c_void_p, c_int64] + [c_void_p] * 8 + [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64]
        + [c_void_p] * 8 + [c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "th_mse_grad": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_int, c_void_p]),
    "th_adam_step": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_float, c_float, c_float, c_int, c_float, c_int,
         c_int, c_void_p, c_void_p],
    ),
    "th_scale_cast": (c_int, [c_void_p, c_void_p, c_int64, c_float, c_int, c_void_p]),
    "th_launch_count": (ctypes.c_longlong, []),
}  # fmt: skip


class KernelTimer:
    r"""Collects CUDA-event timings of every launching C-ABI call made while it is active.

    Events are recorded on the stream the call launches on (torch's current stream), directly
    before and after the call, so the difference is the device time of the kernels that call
    queued.  ``summary()`` synchronises and returns ``{entry point: (calls, total ms)}``.
    """

    LAUNCHING = ("th_field_fwd", "th_field_bwd", "th_hash_fwd", "th_hash_bwd", "th_mlp_fwd", "th_mlp_fwd_mse", "th_mlp_bwd", "th_rev_fwd", "th_rev_bwd",
                 "th_mse_grad", "th_adam_step", "th_scale_cast")  # fmt: skip

    def __init__(self):
        self.records = []

    def __enter__(self):
        global _ACTIVE_TIMER
        _ACTIVE_TIMER = self
        return self

    def __exit__(self, *exc):
        global _ACTIVE_TIMER
        _ACTIVE_TIMER = None
        return False

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, start, stop in self.records:
            calls, total = out.get(name, (0, 0.0))
            out[name] = (calls + 1, total + start.elapsed_time(stop))
        return out


_ACTIVE_TIMER: Optional[KernelTimer] = None


class _Library:
    r"""Thin proxy over the ``ctypes.CDLL``: same attribute names, optional event timing."""

    def __init__(self, handle: ctypes.CDLL):
        self._handle = handle
        for name in SIGNATURES:
            raw = getattr(handle, name)
            setattr(self, name, self._timed(name, raw) if name in KernelTimer.LAUNCHING else raw)

    @staticmethod
    def _timed(name, raw):
        def call(*args):
            timer = _ACTIVE_TIMER
            if timer is None:
                return raw(*args)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            code = raw(*args)
            stop.record()
            timer.records.append((name, start, stop))
            return code

        return call


@lru_cache(maxsize=1)
def lib() -> _Library:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build the CUDA extension with `python -m triton_helpers_b200.build` "
            "(there is no fallback path)"
        )
    handle = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return _Library(handle)


def check(code: int, what: str) -> None:
    if code != 0:
        reason = lib().th_last_error_string().decode(errors="replace")
        raise RuntimeError(f"{what} failed with code {code}: {reason}")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(t: Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32, float16 or bfloat16") from None


def ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def i32_array(values: Sequence[int]):
    return (c_int32 * len(values))(*values)


def i64_array(values: Sequence[int]):
    return (c_int64 * len(values))(*values)


def require_cuda(*tensors: Optional[Tensor]) -> torch.device:
    r"""All given tensors must live on one CUDA device (hash_encoding/kernel.py:560-564 of the reference)."""
    devices = {t.device for t in tensors if t is not None}
    assert len(devices) == 1 and all(d.type == "cuda" for d in devices), (
        f"All tensors must be on the same device: {devices}"
    )
    return next(iter(devices))
