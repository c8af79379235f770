r"""Host-side helpers of ``triton_helpers/ops.py`` (:91-129).

The ``@triton.jit`` device helpers of that file (activations, ``high_low_mod`` ...) have no
Python-visible counterpart here: their arithmetic lives in the CUDA sources
(``csrc/mma_tiles.cuh`` for the activations and their derivatives, ``csrc/hash_encoding.cu``
for the non-power-of-two hash modulo, done with 64-bit products like the reference's CPU
path).  The two host helpers keep their signatures; "function" arguments are plain callables
instead of ``triton.JITFunction`` objects.
"""
from importlib import import_module
from typing import Any, Callable, Iterable, Optional, Union


def ensure_str(fn: Union[str, Callable], choices: Optional[Iterable[str]] = None) -> str:
    r"""Return ``fn`` as a string, checking it against ``choices`` when it already is one.

    A callable becomes ``"<module>.<name>"`` (what the reference does for JIT functions, ops.py:91-107).
    """
    if isinstance(fn, str):
        if (choices is not None) and fn not in (allowed := set(choices)):
            raise ValueError(f"Function {fn} not in {allowed}")
        return fn
    return f"{fn.__module__}.{fn.__name__}"


def import_path(path: str) -> Any:
    r"""Import an attribute given its dotted path, e.g. ``"package.module.function"`` (ops.py:110-129)."""
    path = getattr(path, "value", path)
    assert isinstance(path, str)
    module_name, _, attr = path.rpartition(".")
    return getattr(import_module(module_name), attr)
