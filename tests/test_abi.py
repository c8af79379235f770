r"""The C-ABI library builds, loads, and exports every symbol ``include/th_b200.h`` declares.

No compute call is made here (no GPU is needed): argument-validation paths that return
before any CUDA call are exercised instead.
"""
import ctypes
import re
from pathlib import Path

import pytest

from triton_helpers_b200 import _lib, build

HEADER = Path(__file__).resolve().parent.parent / "include" / "th_b200.h"


@pytest.fixture(scope="module")
def library():
    if not _lib.LIB_PATH.exists():
        build.build()
    return _lib.lib()


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(th_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_families():
    names = declared_symbols()
    assert "th_version" in names and "th_last_error_string" in names
    assert {"th_hash_fwd", "th_hash_bwd", "th_hash_debug_indices"} <= set(names)


def test_every_declared_symbol_is_exported_and_bound(library):
    for name in declared_symbols():
        assert hasattr(library, name), f"{name} is declared in th_b200.h but not exported by the library"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature in triton_helpers_b200/_lib.py"
    assert set(_lib.SIGNATURES) == set(declared_symbols())


def test_version_and_error_text(library):
    assert library.th_version() >= 2
    assert isinstance(library.th_last_error_string(), bytes)


def test_argument_errors_are_reported_without_touching_a_gpu(library):
    res = _lib.i32_array([16, 32])
    rows = _lib.i64_array([17**3, 2**14])
    offs = _lib.i64_array([0, 17**3])
    primes = _lib.i64_array([1, 2654435761, 805459861])
    # 40 levels: more than TH_MAX_LEVELS
    rc = library.th_hash_fwd(None, 3, 1, 0, None, 0, None, 4, 10, 3, 2, 40, res, rows, offs, primes, 1.0, 0, 40, None)
    assert rc == -1 and b"n_levels" in library.th_last_error_string()
    # four coordinate dimensions
    rc = library.th_hash_fwd(None, 4, 1, 0, None, 0, None, 4, 10, 4, 2, 2, res, rows, offs, primes, 1.0, 0, 2, None)
    assert rc == -2
    # null pointers with a non-empty batch
    rc = library.th_hash_fwd(None, 3, 1, 0, None, 0, None, 4, 10, 3, 2, 2, res, rows, offs, primes, 1.0, 0, 2, None)
    assert rc == -1 and b"null" in library.th_last_error_string()
    # empty batch is a successful no-op
    rc = library.th_hash_bwd(None, 3, 1, 0, None, 4, None, 0, 0, 3, 2, 2, res, rows, offs, primes, 1.0, 0, 2, None)
    assert rc == 0
    # bad level range
    rc = library.th_hash_bwd(None, 3, 1, 0, None, 4, None, 0, 10, 3, 2, 2, res, rows, offs, primes, 1.0, 1, 1, None)
    assert rc == -1 and b"level range" in library.th_last_error_string()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libth_b200.so")
    _lib.lib.cache_clear()
    try:
        with pytest.raises(RuntimeError, match="no fallback"):
            _lib.lib()
    finally:
        _lib.lib.cache_clear()
