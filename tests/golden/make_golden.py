r"""Writes ``tests/golden/hash_reference.npz`` by RUNNING THE REFERENCE's own CPU functions.

Run once, in a checkout that has the reference tree next to it::

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/triton-helpers

The reference cannot be installed (``triton_helpers/__init__.py:12`` asks importlib for the
version of an installed distribution), so the script puts the tree on ``sys.path`` and
answers that one metadata query itself.  Only ``_cpu_*`` functions and ``helpers.py`` are
called; no Triton kernel is launched.

What is stored (inputs AND outputs, so the tests never depend on a torch RNG stream):

* ``geom/<name>/{res,rows,offsets,first_hash}`` - level geometry for the benchmark
  configurations and the shapes of the reference's own tests;
* ``lookup/<i>/{x,idx}`` + parameters - ``_cpu_embedding_lookup`` on the cases of
  ``tests/test_layers/test_hash_encoding.py:307-370``;
* ``interp/{x,e,out}`` - ``_cpu_interpolate`` as in ``test_hash_encoding.py:156-172``;
* ``enc/<i>/{x,table,out,grad_out,grad_table}`` - ``_cpu_hash_encoding`` forward and the
  autograd table gradient on small tables, float32 and float16.
"""
import importlib.metadata as md
import os
import sys

import numpy as np
import torch


def load_reference(root: str):
    sys.path.insert(0, root)
    real = md.version
    md.version = lambda name: "0.0.0" if name == "triton-helpers" else real(name)
    import warnings

    warnings.simplefilter("ignore")
    from triton_helpers.layers.hash_encoding import helpers, kernel

    return kernel, helpers


GEOMETRIES = {
    # name: (L, T, D, N_min, N_max)
    "cfg0": (16, 2**19, 3, 16, 2048),
    "cfg4": (16, 2**22, 3, 16, 4096),
    "default": (16, 2**14, 3, 16, 512),
    "t20": (16, 2**20, 3, 16, 512),
    "d2_small": (2, 25, 2, 2, 4),
    "d2_l8": (8, 81, 2, 2, 128),
    "nonpow2": (8, 5000, 3, 4, 96),
}

LOOKUPS = [
    # (L, D, N_level, T)   -- tests/test_layers/test_hash_encoding.py:307-370
    (4, 3, 8, 9**3), (4, 3, 8, 9**3 - 2), (4, 3, 8, 1024), (4, 3, 8, 256),
    (64, 2, 16, 17**2), (64, 3, 16, 17**2), (64, 3, 16, 17**2 - 2),
    (64, 3, 128, 129**2), (64, 3, 128, 129**2 - 1),
    (64, 3, 100, 129**2), (64, 3, 100, 129**2 - 1), (64, 3, 101, 1048576),
    (64, 3, 2048, 2**19), (64, 3, 4096, 2**22), (64, 1, 37, 64),
]

ENCODINGS = [
    # (N, D, F, T, L, N_min, N_max, dtype)
    (4, 2, 2, 25, 2, 2, 4, "float32"),
    (4, 2, 2, 81, 8, 2, 128, "float32"),
    (100, 3, 2, 2**10, 8, 16, 256, "float32"),
    (100, 3, 2, 2**10, 8, 16, 256, "float16"),
    (64, 3, 4, 1000, 4, 4, 64, "float32"),
    (33, 3, 2, 2**12, 16, 16, 512, "float16"),
    (50, 1, 2, 1024, 4, 8, 256, "float32"),
]


def main(root: str) -> None:
    kernel, helpers = load_reference(root)
    out = {}
    for name, (L, T, D, lo, hi) in GEOMETRIES.items():
        out[f"geom/{name}/params"] = np.array([L, T, D, lo, hi], dtype=np.int64)
        out[f"geom/{name}/res"] = np.array(helpers.compute_resolutions(L, lo, hi), dtype=np.int64)
        out[f"geom/{name}/rows"] = np.array(helpers.compute_embedding_counts(L, T, D, lo, hi), dtype=np.int64)
        out[f"geom/{name}/offsets"] = np.array(
            [helpers.compute_level_embedding_offset(i, L, T, D, lo, hi) for i in range(L)], dtype=np.int64
        )
        out[f"geom/{name}/first_hash"] = np.array(helpers.get_first_hash_level(lo, hi, L, T, D), dtype=np.int64)
        out[f"geom/{name}/b"] = np.array(helpers.compute_b(lo, hi, L), dtype=np.float64)

    pi = torch.tensor([kernel.PI_1, kernel.PI_2, kernel.PI_3], dtype=torch.int64)
    torch.manual_seed(0)
    for i, (L, D, res, T) in enumerate(LOOKUPS):
        x = torch.rand(L, D)
        x[0] = 0.0
        if D == 3:
            # the closed upper end passes the reference's range assert (kernel.py:116); for D < 3 the
            # dense index of the all-ones corner is one past the level, so only D = 3 stores it
            x[-1] = 1.0
        rows = min((res + 1) ** D, T)
        idx = kernel._cpu_embedding_lookup(x, pi[:D], D, rows, res)
        out[f"lookup/{i}/params"] = np.array([L, D, res, rows], dtype=np.int64)
        out[f"lookup/{i}/x"] = x.numpy()
        out[f"lookup/{i}/idx"] = idx.numpy()

    x = torch.rand(40, 3)
    e = torch.randn(40, 8, 2)
    out["interp/x"], out["interp/e"] = x.numpy(), e.numpy()
    out["interp/out"] = kernel._cpu_interpolate(x, e, 3, 1).numpy()
    out["interp/out_res7"] = kernel._cpu_interpolate(x, e, 3, 7).numpy()

    for i, (N, D, F, T, L, lo, hi, dt) in enumerate(ENCODINGS):
        dtype = getattr(torch, dt)
        rows = helpers.compute_embedding_counts(L, T, D, lo, hi)
        table = torch.randn(sum(rows), F).to(dtype).requires_grad_(True)
        x = torch.rand(N, D)
        o = torch.zeros(N, F * L, dtype=dtype)
        o = kernel._cpu_hash_encoding(x, table, pi[:D], o, D, F, T, L, lo, hi)
        grad_out = torch.randn(N, F * L).to(dtype)
        o.backward(grad_out)
        out[f"enc/{i}/params"] = np.array([N, D, F, T, L, lo, hi], dtype=np.int64)
        out[f"enc/{i}/dtype"] = np.array(dt)
        out[f"enc/{i}/x"] = x.numpy()
        out[f"enc/{i}/table"] = table.detach().float().numpy().astype(np.float16 if dt == "float16" else np.float32)
        out[f"enc/{i}/out"] = o.detach().float().numpy()
        out[f"enc/{i}/grad_out"] = grad_out.float().numpy()
        out[f"enc/{i}/grad_table"] = table.grad.float().numpy()
    out["counts"] = np.array([len(LOOKUPS), len(ENCODINGS)], dtype=np.int64)

    dest = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hash_reference.npz")
    np.savez_compressed(dest, **out)
    print(f"wrote {dest}: {os.path.getsize(dest) / 1024:.1f} KiB, {len(out)} arrays")


if __name__ == "__main__":
    main(sys.argv[1])
