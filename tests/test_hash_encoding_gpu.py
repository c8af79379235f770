r"""Parity of the CUDA hash encoding with the CPU oracle and the reference's golden vectors.

Every test goes through the Python layer, which calls the C ABI (``th_hash_fwd`` /
``th_hash_bwd`` / ``th_hash_debug_indices``) with no other compute path available.
Tolerances (the benchmark specification): indices bit-exact; float32 forward ``max|a-b| / max|b|
<= 1e-6``; float32 table gradient ``<= 1e-5`` (atomics reorder the sums); float16 tables
use the reference's own test tolerances (``atol=1e-2`` forward,
``atol=1e-3*N, rtol=1e-2`` backward; tests/test_layers/test_hash_encoding.py:432,489).
"""
import numpy as np
import pytest
import torch

from oracle import hash_encoding as oracle
from triton_helpers_b200.layers.hash_encoding import HashEncoding, hash_encoding
from triton_helpers_b200.layers.hash_encoding.helpers import (
    compute_embedding_counts,
    compute_resolutions,
    get_first_hash_level,
    level_geometry,
)
from triton_helpers_b200.layers.hash_encoding.kernel import hash_corner_indices

pytestmark = pytest.mark.gpu

FWD_TOL_F32 = 1e-6
BWD_TOL_F32 = 1e-5

QUADRANT_POINTS = [[0, 0], [0.55, 0.55], [0.45, 0.45], [0.9999, 0.9999], [0.55, 0.45], [0.45, 0.55]]
QUADRANT_DENSE = [[0, 1, 2, 3], [3, 4, 5, 6], [0, 1, 2, 3], [3, 4, 5, 6], [1, 2, 3, 4], [2, 3, 4, 5]]
QUADRANT_HASHED = [[0, 1, 5, 4], [4, 0, 4, 1], [0, 1, 5, 4], [4, 0, 4, 1], [1, 2, 4, 0], [5, 4, 3, 4]]


def nerr(got: torch.Tensor, want: torch.Tensor) -> float:
    r"""max|got - want| / max|want| in float64."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-300))


def make_case(N, D, F, T, L, lo, hi, dtype, seed=0, clustered=False):
    g = torch.Generator().manual_seed(seed)
    rows = compute_embedding_counts(L, T, D, lo, hi)
    table = (torch.rand(sum(rows), F, generator=g) * 2 - 1).mul(1e-1).to(dtype)
    if clustered:
        centres = torch.rand(8, D, generator=g) * 0.6 + 0.2
        which = torch.randint(0, 8, (N,), generator=g)
        x = centres[which] + 0.02 * torch.randn(N, D, generator=g)
        x = x.clamp(0, 1 - 2**-24)
    else:
        x = torch.rand(N, D, generator=g)
    go = torch.randn(N, L * F, generator=g).to(dtype)
    return x, table, go, dict(table_cap=T, levels=L, n_min=lo, n_max=hi)


# ---- indices and weights: bit exact ----------------------------------------------------------


@pytest.mark.parametrize("rows,expected", [(9, QUADRANT_DENSE), (7, QUADRANT_HASHED)])
def test_known_answer_index_tables(rows, expected):
    x = torch.tensor(QUADRANT_POINTS, dtype=torch.float32, device="cuda")
    idx, _ = hash_corner_indices(x, [2], [rows])
    assert idx[:, 0].cpu().tolist() == expected


def test_indices_match_reference_fixtures(golden):
    for i in range(int(golden["counts"][0])):
        L, D, res, rows = (int(v) for v in golden[f"lookup/{i}/params"])
        x = torch.from_numpy(golden[f"lookup/{i}/x"]).cuda()
        idx, _ = hash_corner_indices(x, [res], [rows])
        assert np.array_equal(idx[:, 0].cpu().numpy(), golden[f"lookup/{i}/idx"]), f"lookup case {i}"


@pytest.mark.parametrize("name", ["cfg0", "cfg4", "default", "nonpow2", "d2_l8"])
def test_indices_and_weights_bit_exact_all_levels(golden, name):
    L, T, D, lo, hi = (int(v) for v in golden[f"geom/{name}/params"])
    res, rows = golden[f"geom/{name}/res"].tolist(), golden[f"geom/{name}/rows"].tolist()
    g = torch.Generator().manual_seed(3)
    x = torch.rand(5000, D, generator=g)
    x[0] = 0.0
    x[1] = 1 - 2**-24
    idx, w = hash_corner_indices(x.cuda(), res, rows)
    for lvl in range(L):
        want_idx = oracle.corner_indices(x, oracle.PRIMES, D, rows[lvl], res[lvl])
        want_w = oracle.corner_weights(x, D, res[lvl])
        assert torch.equal(idx[:, lvl].cpu(), want_idx), f"{name} level {lvl} indices"
        assert torch.equal(w[:, lvl].cpu(), want_w), f"{name} level {lvl} weights"
        assert int(idx[:, lvl].min()) >= 0 and int(idx[:, lvl].max()) < rows[lvl]


def test_indices_fp16_coords_and_scale():
    g = torch.Generator().manual_seed(5)
    x = torch.rand(777, 3, generator=g).half()
    res, rows = [16, 101, 512], [17**3, 2**14, 2**14]
    idx, w = hash_corner_indices((x * 2).cuda(), res, rows, scale=2.0)
    for lvl in range(3):
        assert torch.equal(idx[:, lvl].cpu(), oracle.corner_indices(x.float(), oracle.PRIMES, 3, rows[lvl], res[lvl]))
        assert torch.equal(w[:, lvl].cpu(), oracle.corner_weights(x.float(), 3, res[lvl]))


@pytest.mark.parametrize("scale", [3.0, 0.7, 1000.0])
def test_indices_with_a_scale_that_is_not_a_power_of_two(scale):
    # The kernels divide the coordinate by `scale` (one float32 division) and then follow the CPU path, which
    # is what the reference's tests do before calling its CPU function (tests/test_layers/test_hash_encoding.py:427-428):
    # bit-exact against the oracle fed x / scale.  (The reference's Triton kernel folds 1 / scale into its first
    # level multiplier instead and can land in the neighbouring cell on a cell boundary.)
    g = torch.Generator().manual_seed(9)
    x = torch.rand(5000, 3, generator=g) * scale
    res, rows = [16, 23, 101, 512, 4096], [17**3, 24**3, 2**14, 2**19, 2**22]
    idx, w = hash_corner_indices(x.cuda(), res, rows, scale=scale)
    unit = x / scale  # float32 division, as in the kernels
    for lvl in range(len(res)):
        assert torch.equal(idx[:, lvl].cpu(), oracle.corner_indices(unit, oracle.PRIMES, 3, rows[lvl], res[lvl]))
        assert torch.equal(w[:, lvl].cpu(), oracle.corner_weights(unit, 3, res[lvl]))


@pytest.mark.parametrize("res", [16, 32, 512])
@pytest.mark.parametrize("unique", [False, True])
def test_indices_in_range(res, unique):
    # reference TestEmbeddingLookup.test_overflow
    g = torch.Generator().manual_seed(0)
    rows = (res + 1) ** 3 - (0 if unique else 2)
    x = torch.rand(499, 3, generator=g).cuda()
    idx, _ = hash_corner_indices(x, [res], [rows])
    assert int(idx.min()) >= 0 and int(idx.max()) < rows


# ---- forward ---------------------------------------------------------------------------------


def test_forward_matches_reference_fixtures(golden):
    for i in range(int(golden["counts"][1])):
        N, D, F, T, L, lo, hi = (int(v) for v in golden[f"enc/{i}/params"])
        dtype = getattr(torch, str(golden[f"enc/{i}/dtype"]))
        x = torch.from_numpy(golden[f"enc/{i}/x"]).cuda()
        table = torch.from_numpy(golden[f"enc/{i}/table"]).to(dtype).cuda()
        want = torch.from_numpy(golden[f"enc/{i}/out"])
        got = hash_encoding(x, table, None, None, T, lo, hi, L)
        assert got.dtype == dtype and got.shape == (N, L * F)
        if dtype == torch.float32:
            assert nerr(got, want) <= FWD_TOL_F32, f"encoding case {i}"
        else:
            torch.testing.assert_close(got.float().cpu(), want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize(
    "N,D,F,T,L,lo,hi",
    [
        (65536, 3, 2, 2**19, 16, 16, 2048),  # benchmark configuration 0
        (10001, 3, 4, 2**16, 16, 16, 4096),
        (4099, 2, 2, 2**12, 8, 4, 512),
        (1000, 1, 1, 2**10, 4, 8, 256),
        (3000, 3, 8, 5000, 8, 4, 96),  # hashed levels with a row count that is not a power of two
        (2048, 3, 1, 2**14, 2, 16, 512),
    ],
)
def test_forward_backward_float32_against_oracle(N, D, F, T, L, lo, hi):
    x, table, go, kw = make_case(N, D, F, T, L, lo, hi, torch.float32)
    want = oracle.encode(x, table, oracle.PRIMES[:D], **kw)
    want_grad = oracle.encode_backward(x, go, table, oracle.PRIMES[:D], **kw)
    t = table.cuda().requires_grad_(True)
    got = hash_encoding(x.cuda(), t, None, None, T, lo, hi, L)
    assert nerr(got, want) <= FWD_TOL_F32
    got.backward(go.cuda())
    assert t.grad.shape == table.shape and t.grad.dtype == torch.float32
    assert nerr(t.grad, want_grad) <= BWD_TOL_F32


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_forward_backward_half_tables_against_oracle(dtype):
    N, D, F, T, L, lo, hi = 20000, 3, 2, 2**14, 16, 16, 512
    x, table, go, kw = make_case(N, D, F, T, L, lo, hi, dtype)
    want = oracle.encode(x, table, **kw)
    want_grad = oracle.encode_backward(x, go, table, **kw)  # float32 sums, one rounding
    t = table.cuda().requires_grad_(True)
    got = hash_encoding(x.cuda(), t, None, None, T, lo, hi, L)
    assert got.dtype == dtype
    # forward: one rounding of a float32 sum, so at most one ulp from the oracle
    torch.testing.assert_close(got.float().cpu(), want.float(), atol=1e-3, rtol=1e-2)
    got.backward(go.cuda())
    # backward: half-precision atomics round every partial sum
    assert nerr(t.grad, want_grad) <= (2e-2 if dtype == torch.float16 else 1e-1)


@pytest.mark.parametrize(
    "N,D,F,T,L,lo,hi,scale",
    [
        (4, 2, 2, 25, 2, 2, 4, 1.0),
        (4, 2, 2, 81, 8, 2, 128, 1.0),
        (4, 3, 2, 2**14, 16, 16, 512, 1.0),
        (100, 3, 2, 2**14, 16, 16, 512, 1.0),
        (100, 3, 2, 2**20, 16, 16, 512, 1.0),
        (100, 3, 2, 2**14, 16, 16, 512, 2.0),
    ],
)
def test_reference_forward_cases_fp16_tables(N, D, F, T, L, lo, hi, scale):
    # shapes, seed and tolerance of the reference's TestHashEncoding.test_forward_torch_baseline
    torch.random.manual_seed(0)
    rows = compute_embedding_counts(L, T, D, lo, hi)
    e = torch.randn(sum(rows), F, dtype=torch.float16)
    x = torch.rand(N, D)
    want = oracle.encode(x, e, oracle.PRIMES[:D], table_cap=T, levels=L, n_min=lo, n_max=hi)
    got = hash_encoding((x * scale).cuda(), e.cuda(), None, None, T, lo, hi, L, scale=scale)
    hash_level = min(get_first_hash_level(lo, hi, L, T, D), L)
    torch.testing.assert_close(got[..., hash_level * F :].cpu(), want[..., hash_level * F :], atol=1e-2, rtol=0)
    torch.testing.assert_close(got.cpu(), want, atol=1e-2, rtol=0)


@pytest.mark.parametrize(
    "N,D,F,T,L,lo,hi,scale",
    [(65536, 3, 2, 2**20, 16, 16, 512, 1.0), (128 * 1024, 3, 2, 2**14, 16, 16, 512, 1.0), (100, 3, 2, 2**14, 16, 16, 512, 2.0)],
)
def test_reference_backward_cases_fp16_tables(N, D, F, T, L, lo, hi, scale):
    # shapes, seed and tolerance of the reference's TestHashEncoding.test_backward_torch_baseline
    torch.random.manual_seed(0)
    rows = compute_embedding_counts(L, T, D, lo, hi)
    e = torch.randn(sum(rows), F, dtype=torch.float16)
    x = torch.rand(N, D)
    go = torch.ones(N, L * F, dtype=torch.float16)  # the reference back-propagates o.sum()
    want = oracle.encode_backward(x, go, e, oracle.PRIMES[:D], table_cap=T, levels=L, n_min=lo, n_max=hi)
    t = e.cuda().requires_grad_(True)
    hash_encoding((x * scale).cuda(), t, None, None, T, lo, hi, L, scale=scale).sum().backward()
    torch.testing.assert_close(t.grad.cpu().float(), want.float(), atol=1e-3 * N, rtol=1e-2)


# ---- edge cases ------------------------------------------------------------------------------


def test_empty_single_and_ragged_batches():
    D, F, T, L, lo, hi = 3, 2, 2**12, 8, 16, 256
    for N in (0, 1, 255, 256, 257, 1023):
        x, table, go, kw = make_case(max(N, 1), D, F, T, L, lo, hi, torch.float32, seed=N)
        x, go = x[:N], go[:N]
        t = table.cuda().requires_grad_(True)
        got = hash_encoding(x.cuda(), t, None, None, T, lo, hi, L)
        assert got.shape == (N, L * F)
        got.backward(go.cuda())
        if N == 0:
            assert float(t.grad.abs().max()) == 0.0
            continue
        assert nerr(got, oracle.encode(x, table, **kw)) <= FWD_TOL_F32
        assert nerr(t.grad, oracle.encode_backward(x, go, table, **kw)) <= BWD_TOL_F32


def test_leading_dims_features_and_strided_inputs():
    D, F, T, L, lo, hi = 3, 2, 2**12, 8, 16, 256
    x, table, go, kw = make_case(6 * 50, D, F, T, L, lo, hi, torch.float32, seed=7)
    feats = torch.randn(6, 50, 5)
    want = oracle.encode(x, table, **kw).view(6, 50, L * F)
    # coordinates that are a strided view (every other column of a wider buffer)
    wide = torch.zeros(6, 50, 2 * D).cuda()
    wide[..., ::2] = x.view(6, 50, D).cuda()
    got = hash_encoding(wide[..., ::2], table.cuda(), feats.cuda(), None, T, lo, hi, L)
    assert got.shape == (6, 50, L * F + 5)
    assert nerr(got[..., : L * F], want) <= FWD_TOL_F32
    assert torch.equal(got[..., L * F :].cpu(), feats)
    # gradient through the feature-extended output: only the table columns matter
    t = table.cuda().requires_grad_(True)
    out = hash_encoding(x.view(6, 50, D).cuda(), t, feats.cuda(), None, T, lo, hi, L)
    full_go = torch.cat([go.view(6, 50, -1), torch.randn(6, 50, 5)], -1).cuda()
    out.backward(full_go)
    assert nerr(t.grad, oracle.encode_backward(x, go, table, **kw)) <= BWD_TOL_F32


@pytest.mark.parametrize("divider", [1, 2, 4, 8])
def test_divider_passes_give_the_same_result(divider):
    D, F, T, L, lo, hi = 3, 2, 2**12, 8, 16, 256
    x, table, go, kw = make_case(3000, D, F, T, L, lo, hi, torch.float32, seed=9)
    t = table.cuda().requires_grad_(True)
    ref = hash_encoding(x.cuda(), table.cuda(), None, None, T, lo, hi, L)
    got = hash_encoding(x.cuda(), t, None, None, T, lo, hi, L, divider=divider, bwd_divider=divider)
    assert torch.equal(got, ref)
    got.backward(go.cuda())
    assert nerr(t.grad, oracle.encode_backward(x, go, table, **kw)) <= BWD_TOL_F32


def test_argument_checks_match_the_reference():
    x = torch.rand(10, 3, device="cuda")
    table = torch.randn(sum(compute_embedding_counts(16, 2**14, 3, 16, 512)), 2, device="cuda")
    with pytest.raises(AssertionError, match="power of 2"):
        hash_encoding(x, table, levels=12)
    with pytest.raises(AssertionError, match="Divider"):
        hash_encoding(x, table, divider=3)
    with pytest.raises(AssertionError, match="Gradients not supported for coords"):
        hash_encoding(x.clone().requires_grad_(True), table)
    with pytest.raises(AssertionError, match="same device"):
        hash_encoding(x.cpu(), table)
    with pytest.raises(ValueError, match="Pi must be provided"):
        hash_encoding(torch.rand(10, 4, device="cuda"), table)
    with pytest.raises(AssertionError, match="Coords must be float"):
        hash_encoding(torch.zeros(10, 3, device="cuda", dtype=torch.int32), table)


# ---- contention: clustered points hit the warp-aggregated path ---------------------------------


@pytest.mark.parametrize("dtype,F", [(torch.float32, 4), (torch.float32, 2), (torch.float16, 2)])
def test_backward_clustered_points(dtype, F):
    N, D, T, L, lo, hi = 30000, 3, 2**15, 16, 16, 4096
    x, table, go, kw = make_case(N, D, F, T, L, lo, hi, dtype, seed=11, clustered=True)
    want = oracle.encode_backward(x, go, table, **kw)
    t = table.cuda().requires_grad_(True)
    hash_encoding(x.cuda(), t, None, None, T, lo, hi, L).backward(go.cuda())
    assert nerr(t.grad, want) <= (BWD_TOL_F32 if dtype == torch.float32 else 2e-2)


def test_contention_configuration_on_its_own_table():
    # benchmark configuration 4's table as it is - 16 levels x 4 float32 features, T = 2^22, 16..4096, 42 585 337
    # rows (681 MB) - with 65 536 points drawn from its mixture of 8 Gaussians: forward within 1e-6 and table
    # gradient within 1e-5 of the oracle (the size the oracle finishes in seconds; the full 2^22 points are
    # covered by the size-independent properties below)
    N, D, F, T, L, lo, hi = 65536, 3, 4, 2**22, 16, 16, 4096
    x, table, go, kw = make_case(N, D, F, T, L, lo, hi, torch.float32, seed=17, clustered=True)
    assert table.shape == (42_585_337, 4)
    want = oracle.encode(x, table, **kw)
    want_grad = oracle.encode_backward(x, go, table, **kw)
    t = table.cuda().requires_grad_(True)
    out = hash_encoding(x.cuda(), t, None, None, T, lo, hi, L)
    assert nerr(out, want) <= FWD_TOL_F32
    out.backward(go.cuda())
    assert nerr(t.grad, want_grad) <= BWD_TOL_F32
    # the gradient touches only rows the oracle touches
    assert torch.equal((t.grad != 0).any(1).cpu(), (want_grad != 0).any(1))


def test_backward_all_points_identical():
    # every lane of every warp in the same cell at every level: the longest aggregation chains
    N, D, F, T, L, lo, hi = 4096 + 37, 3, 2, 2**12, 8, 16, 256
    _, table, go, kw = make_case(N, D, F, T, L, lo, hi, torch.float32, seed=13)
    x = torch.tensor([[0.3141, 0.2718, 0.5772]]).repeat(N, 1)
    want = oracle.encode_backward(x, go, table, **kw)
    t = table.cuda().requires_grad_(True)
    hash_encoding(x.cuda(), t, None, None, T, lo, hi, L).backward(go.cuda())
    assert nerr(t.grad, want) <= BWD_TOL_F32


# ---- large batches: the coarsest dense levels are accumulated in shared memory -------------------


@pytest.mark.parametrize(
    "D,F,T,L,lo,hi,dtype",
    [
        (3, 2, 2**19, 16, 16, 2048, torch.float32),
        (3, 4, 2**15, 8, 16, 512, torch.float32),
        (2, 2, 2**19, 8, 16, 1024, torch.float32),  # 2-D: every level dense, several fit
        (3, 1, 2**14, 4, 4, 64, torch.float32),
        (3, 2, 2**19, 16, 16, 2048, torch.float16),
        (3, 8, 2**14, 4, 16, 128, torch.bfloat16),
        (3, 8, 2**14, 4, 16, 128, torch.float32),  # 32-byte rows: two 16-byte compare-and-swaps
        (3, 4, 2**14, 4, 16, 128, torch.float16),  # 8-byte rows
        (3, 1, 2**14, 4, 16, 64, torch.float16),  # 2-byte rows: native half add
        (3, 4, 2**21, 8, 16, 1024, torch.float32),  # 144 MB of levels: cut into cache-sized passes
    ],
)
def test_large_batch_against_oracle(D, F, T, L, lo, hi, dtype):
    N = 2**18 + 37
    x, table, go, kw = make_case(N, D, F, T, L, lo, hi, dtype, seed=17)
    want_out = oracle.encode(x, table, **kw)
    want = oracle.encode_backward(x, go, table, **kw)
    t = table.cuda().requires_grad_(True)
    out = hash_encoding(x.cuda(), t, None, None, T, lo, hi, L)
    if dtype == torch.float32:
        assert nerr(out, want_out) <= FWD_TOL_F32
    else:
        torch.testing.assert_close(out.float().cpu(), want_out.float(), atol=1e-3, rtol=1e-2)
    out.backward(go.cuda())
    if dtype == torch.float32:
        assert nerr(t.grad, want) <= BWD_TOL_F32
    else:
        torch.testing.assert_close(t.grad.float().cpu(), want.float(), atol=1e-3 * N, rtol=1e-2)
        assert nerr(t.grad, want) <= (2e-2 if dtype == torch.float16 else 1e-1)


@pytest.mark.parametrize("divider", [1, 2, 4])
def test_backward_large_batch_equals_the_sum_of_its_halves(divider):
    # the halves are below the batch size at which shared-memory accumulation starts
    N, D, F, T, L, lo, hi = 2**18, 3, 2, 2**17, 8, 16, 512
    x, table, go, _ = make_case(N, D, F, T, L, lo, hi, torch.float32, seed=19)
    x, go = x.cuda(), go.cuda()

    def grad(xs, gs):
        t = table.cuda().requires_grad_(True)
        hash_encoding(xs, t, None, None, T, lo, hi, L, divider, divider).backward(gs)
        return t.grad

    whole = grad(x, go)
    halves = grad(x[: N // 2], go[: N // 2]) + grad(x[N // 2 :], go[N // 2 :])
    assert nerr(whole, halves) <= BWD_TOL_F32


# ---- size-independent properties at full benchmark sizes ---------------------------------------


@pytest.mark.parametrize(
    "N,F,T,hi,dtype",
    [(2**21, 2, 2**19, 2048, torch.float16), (2**20, 4, 2**22, 4096, torch.float32)],
)
def test_partition_of_unity_and_gradient_mass_at_full_size(N, F, T, hi, dtype):
    # table of ones -> every output is 1 (corner weights sum to 1); gradient of the table sums,
    # per level and feature, to the column sums of grad_out.  Linearity: bwd(a) + bwd(b) = bwd(a + b).
    L, D, lo = 16, 3, 16
    geo = level_geometry(L, T, D, lo, hi)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.rand(N, D, device="cuda", generator=g)
    table = torch.ones(geo.total_rows, F, device="cuda", dtype=dtype, requires_grad=True)
    out = hash_encoding(x, table, None, None, T, lo, hi, L)
    assert float((out.float() - 1).abs().max()) <= (1e-6 if dtype == torch.float32 else 1e-3)
    if dtype != torch.float32:
        return
    go_a = torch.randn(N, L * F, device="cuda", generator=g)
    go_b = torch.randn(N, L * F, device="cuda", generator=g)
    (grad_a,) = torch.autograd.grad(out, table, go_a, retain_graph=True)
    (grad_b,) = torch.autograd.grad(out, table, go_b, retain_graph=True)
    (grad_ab,) = torch.autograd.grad(out, table, go_a + go_b)
    assert nerr(grad_a + grad_b, grad_ab) <= 1e-4
    for lvl in (0, 5, 15):
        rows = slice(geo.offsets[lvl], geo.offsets[lvl] + geo.rows[lvl])
        mass = grad_a[rows].double().sum(0)
        want = go_a[:, lvl * F : (lvl + 1) * F].double().sum(0)
        assert float((mass - want).abs().max()) <= 1e-3 * float(go_a.abs().double().sum(0).max())


# ---- module ------------------------------------------------------------------------------------


def test_module_autocast_and_state_dict():
    torch.manual_seed(0)
    layer = HashEncoding(2**8, 4, 3, 2, 16, 512).cuda()
    assert set(layer.state_dict().keys()) == {"embeddings", "pi"}
    assert layer.pi.dtype == torch.int64 and layer.embeddings.shape == (sum(compute_embedding_counts(4, 2**8, 3, 16, 512)), 2)
    x = torch.rand(16, 40, 3, device="cuda", requires_grad=True)
    with torch.autocast(device_type="cuda", dtype=torch.float16):
        o = layer(x)
    assert o.dtype == torch.float16 and o.shape == (16, 40, 8)
    o.sum().backward()
    assert layer.embeddings.grad is not None and layer.embeddings.grad.dtype == torch.float32
    # float32 call outside autocast matches the oracle
    with torch.no_grad():
        o32 = layer(x.detach())
    want = oracle.encode(x.detach().cpu().view(-1, 3), layer.embeddings.detach().cpu(), table_cap=2**8, levels=4, n_min=16, n_max=512)
    assert nerr(o32.view(-1, 8), want) <= FWD_TOL_F32
    assert compute_resolutions(4, 16, 512)[0] == 16
