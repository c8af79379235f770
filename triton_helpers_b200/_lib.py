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
    "th_mlp_fwd": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "th_mlp_workspace_bytes": (c_int64, [c_int, c_int, c_int, c_int]),
    "th_mlp_bwd": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "th_rev_fwd": (
        c_int,
        [c_void_p, c_int64] + [c_void_p] * 8 + [c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
    "th_rev_workspace_bytes": (c_int64, [c_int64, c_int, c_int, c_int]),
    "th_rev_bwd": (
        c_int,
        [c_void_p, c_int64] + [c_void_p] * 8 + [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64]
        + [c_void_p] * 8 + [c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ),
}  # fmt: skip


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
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
    return handle


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
