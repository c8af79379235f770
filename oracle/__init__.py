r"""CPU oracle for the three fused operators.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this directory.  The only callers are the
tests, the GPU smoke check and the CPU-baseline / reference arms of the benchmark,
and there it is the checker or the thing timed *beside* the CUDA path, never a
fallback for it.

* ``oracle.hash_encoding`` restates, in plain torch-on-CPU code, the reference's own
  CPU path for the multiresolution hash encoding
  (``triton_helpers/layers/hash_encoding/kernel.py:443-502`` and
  ``triton_helpers/layers/hash_encoding/helpers.py:12-115``).  Parity is PINNED: the
  restatement is checked against the golden index tables the reference's tests hold
  (``tests/test_layers/test_hash_encoding.py:240-251,285-296``) and against fixtures
  produced by importing and running the reference's ``_cpu_*`` functions
  (``tests/golden/make_golden.py`` in this repository wrote them).
* ``oracle.fused_mlp`` restates the PyTorch MLP the reference's tests and benchmark
  compare against (``tests/test_layers/test_fully_fused_mlp.py:21-35``,
  ``triton_helpers/layers/fully_fused_mlp/__main__.py:40-62``): a chain of
  ``F.linear`` + activation evaluated in float32.  The reference holds no numeric
  vectors for it; values are pinned only relative to torch, as in the reference.
* ``oracle.reversible_mlp`` is the additive-coupling stack evaluated with torch
  autograd and stored activations.  The reference has no such operator, so its
  PARITY IS UNPINNED by the reference; the oracle is the definition.
"""
