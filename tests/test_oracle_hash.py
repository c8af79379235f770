r"""Pins the CPU oracle of the hash encoding.

Two anchors: (1) the known-answer index tables that the reference's own tests hold
(tests/test_layers/test_hash_encoding.py:217-305 of the reference, transcribed below),
(2) fixtures produced by running the reference's ``_cpu_*`` functions
(tests/golden/make_golden.py).  The product's host-side geometry helpers are pinned
against the same fixtures.
"""
import numpy as np
import pytest
import torch

from oracle import hash_encoding as oracle
from triton_helpers_b200.layers.hash_encoding import helpers

QUADRANT_POINTS = [[0, 0], [0.55, 0.55], [0.45, 0.45], [0.9999, 0.9999], [0.55, 0.45], [0.45, 0.55]]
# D=2, res=2, T=9: dense (reference test_quadrants_2d_unique)
QUADRANT_DENSE = [[0, 1, 2, 3], [3, 4, 5, 6], [0, 1, 2, 3], [3, 4, 5, 6], [1, 2, 3, 4], [2, 3, 4, 5]]
# D=2, res=2, T=7: hashed, T not a power of two (reference test_quadrants_2d_nonunique)
QUADRANT_HASHED = [[0, 1, 5, 4], [4, 0, 4, 1], [0, 1, 5, 4], [4, 0, 4, 1], [1, 2, 4, 0], [5, 4, 3, 4]]

GEOMS = ["cfg0", "cfg4", "default", "t20", "d2_small", "d2_l8", "nonpow2"]


def test_corner_offsets_match_reference_fixture_tables():
    assert oracle.corner_offsets(2).tolist() == [[0, 0], [1, 0], [0, 1], [1, 1]]
    assert oracle.corner_offsets(3).tolist() == [
        [0, 0, 0], [1, 0, 0], [0, 1, 0], [1, 1, 0], [0, 0, 1], [1, 0, 1], [0, 1, 1], [1, 1, 1],
    ]  # fmt: skip


@pytest.mark.parametrize("rows,expected", [(9, QUADRANT_DENSE), (7, QUADRANT_HASHED)])
def test_known_answer_index_tables(rows, expected):
    x = torch.tensor(QUADRANT_POINTS, dtype=torch.float32)
    idx = oracle.corner_indices(x, oracle.PRIMES, 2, rows, 2)
    assert idx.tolist() == expected


@pytest.mark.parametrize("name", GEOMS)
def test_geometry_oracle_and_product_helpers(golden, name):
    L, T, D, lo, hi = (int(v) for v in golden[f"geom/{name}/params"])
    res = golden[f"geom/{name}/res"].tolist()
    rows = golden[f"geom/{name}/rows"].tolist()
    offs = golden[f"geom/{name}/offsets"].tolist()
    first = int(golden[f"geom/{name}/first_hash"])
    b = float(golden[f"geom/{name}/b"])
    # oracle restatement
    assert oracle.growth_factor(lo, hi, L) == b
    assert oracle.level_resolutions(L, lo, hi) == res
    assert oracle.level_rows(L, T, D, lo, hi) == rows
    assert oracle.level_offsets(L, T, D, lo, hi) == offs
    assert oracle.first_hash_level(lo, hi, L, T, D) == first
    # host logic shipped in the package
    assert helpers.compute_b(lo, hi, L) == b
    assert helpers.compute_resolutions(L, lo, hi) == res
    assert helpers.compute_embedding_counts(L, T, D, lo, hi) == rows
    assert [helpers.compute_level_embedding_offset(i, L, T, D, lo, hi) for i in range(L)] == offs
    assert helpers.get_first_hash_level(lo, hi, L, T, D) == first
    geo = helpers.level_geometry(L, T, D, lo, hi)
    assert list(geo.resolutions) == res and list(geo.rows) == rows and list(geo.offsets) == offs
    assert geo.first_hash_level == first and geo.total_rows == offs[-1] + rows[-1]


def test_benchmark_geometry_values():
    # the table sizes the benchmark configurations rely on
    geo = helpers.level_geometry(16, 2**19, 3, 16, 2048)
    assert geo.resolutions == (16, 22, 30, 42, 58, 80, 111, 153, 212, 294, 406, 561, 776, 1072, 1482, 2048)
    assert geo.total_rows == 6_098_925 and geo.first_hash_level == 5
    geo = helpers.level_geometry(16, 2**22, 3, 16, 4096)
    assert geo.total_rows == 42_585_337 and geo.first_hash_level == 7


def test_seek_to_level(golden):
    L, T, D, lo, hi = (int(v) for v in golden["geom/nonpow2/params"])
    rows = golden["geom/nonpow2/rows"].tolist()
    e = torch.arange(sum(rows) * 2, dtype=torch.float32).view(-1, 2)
    for lvl in range(L):
        view = helpers.seek_to_level_embeddings(e, lvl, L, T, D, lo, hi)
        start = helpers.compute_level_embedding_offset(lvl, L, T, D, lo, hi)
        assert view.shape == (rows[lvl], 2)
        assert view[0, 0] == start * 2


def test_lookup_matches_reference_outputs(golden):
    n_lookup = int(golden["counts"][0])
    assert n_lookup >= 12
    for i in range(n_lookup):
        L, D, res, rows = (int(v) for v in golden[f"lookup/{i}/params"])
        x = torch.from_numpy(golden[f"lookup/{i}/x"])
        idx = oracle.corner_indices(x, oracle.PRIMES, D, rows, res)
        assert np.array_equal(idx.numpy(), golden[f"lookup/{i}/idx"]), f"lookup case {i}"
        assert int(idx.min()) >= 0 and int(idx.max()) < rows


def test_interpolate_matches_reference_outputs(golden):
    x = torch.from_numpy(golden["interp/x"])
    e = torch.from_numpy(golden["interp/e"])
    assert np.array_equal(oracle.interpolate(x, e, 3, 1).numpy(), golden["interp/out"])
    assert np.array_equal(oracle.interpolate(x, e, 3, 7).numpy(), golden["interp/out_res7"])


def test_interpolation_known_answers():
    # corners and centre (reference TestInterpolate.test_corners / test_mean)
    torch.manual_seed(0)
    e = torch.randn(10, 8, 2)
    for coord, corner in [((0, 0, 0), 0), ((0.9999, 0.9999, 0.9999), 7), ((0.9999, 0.9999, 0), 3)]:
        x = torch.tensor(coord, dtype=torch.float32).repeat(10, 1)
        torch.testing.assert_close(oracle.interpolate(x, e, 3, 1), e[:, corner], rtol=0, atol=1e-3)
    x = torch.full((10, 3), 0.5)
    torch.testing.assert_close(oracle.interpolate(x, e, 3, 1), e.mean(1))


def _enc_case(golden, i):
    N, D, F, T, L, lo, hi = (int(v) for v in golden[f"enc/{i}/params"])
    dtype = getattr(torch, str(golden[f"enc/{i}/dtype"]))
    x = torch.from_numpy(golden[f"enc/{i}/x"])
    table = torch.from_numpy(golden[f"enc/{i}/table"]).to(dtype)
    return dict(x=x, table=table, kw=dict(table_cap=T, levels=L, n_min=lo, n_max=hi), D=D, F=F, dtype=dtype)


def test_encode_forward_matches_reference_outputs(golden):
    for i in range(int(golden["counts"][1])):
        c = _enc_case(golden, i)
        out = oracle.encode(c["x"], c["table"], oracle.PRIMES[: c["D"]], **c["kw"])
        assert out.dtype == c["dtype"]
        assert np.array_equal(out.float().numpy(), golden[f"enc/{i}/out"]), f"encoding case {i}"


def test_encode_backward_matches_reference_autograd(golden):
    for i in range(int(golden["counts"][1])):
        c = _enc_case(golden, i)
        go = torch.from_numpy(golden[f"enc/{i}/grad_out"]).to(c["dtype"])
        ref = torch.from_numpy(golden[f"enc/{i}/grad_table"])
        got = oracle.encode_backward(c["x"], go, c["table"], oracle.PRIMES[: c["D"]], **c["kw"]).float()
        scale = ref.abs().max().clamp_min(1e-30)
        tol = 1e-6 if c["dtype"] == torch.float32 else 2e-3  # fp16 autograd rounds every addend
        assert float((got - ref).abs().max() / scale) <= tol, f"encoding case {i}"


def test_encode_backward_is_autograd_of_encode(golden):
    c = _enc_case(golden, 2)
    table = c["table"].clone().requires_grad_(True)
    go = torch.randn(c["x"].shape[0], c["F"] * c["kw"]["levels"], generator=torch.Generator().manual_seed(1))
    oracle.encode(c["x"], table, **c["kw"]).backward(go)
    got = oracle.encode_backward(c["x"], go, table.detach(), **c["kw"])
    torch.testing.assert_close(got, table.grad, rtol=1e-5, atol=1e-6)
