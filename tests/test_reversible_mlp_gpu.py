r"""Parity of the CUDA reversible MLP with its oracle (torch autograd with stored activations).

The reference has no reversible operator, so parity is defined by ``oracle/reversible_mlp.py``
alone (unpinned by the reference).  Tolerances: outputs and parameter gradients within 1e-2
(float16) / 3e-2 (bfloat16: 8-bit mantissa) normalised error of the float32 computation; the
tight comparison is against the oracle that rounds where the kernels round.  The
size-independent property at the full benchmark size is reconstruction: the backward pass must
recover the stack's input from its output.
"""
import pytest
import torch

from oracle import reversible_mlp as oracle
from triton_helpers_b200.layers.reversible_mlp import (
    ReversibleMLP,
    reversible_mlp,
    reversible_mlp_backward,
    reversible_mlp_forward,
)

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16]
LOOSE = {torch.float16: 1e-2, torch.bfloat16: 3e-2}
TIGHT = {torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


def nerr(got, want) -> float:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-300))


def rows_outside(got, want, tol) -> float:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    err = (got - want).abs().reshape(-1, want.shape[-1]).amax(-1) / want.abs().max().clamp_min(1e-300)
    return float((err > tol).double().mean())


def make_params(blocks, half, hidden, bias, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    u = lambda *shape, fan: ((torch.rand(*shape, generator=g) * 2 - 1) / fan**0.5).to(dtype)  # noqa: E731
    weights = (u(blocks * hidden, half, fan=half), u(blocks * half, hidden, fan=hidden),
               u(blocks * hidden, half, fan=half), u(blocks * half, hidden, fan=hidden))  # fmt: skip
    biases = (u(blocks, hidden, fan=half), u(blocks, half, fan=hidden), u(blocks, hidden, fan=half),
              u(blocks, half, fan=hidden)) if bias else (None,) * 4  # fmt: skip
    return weights, biases


def to_cuda(ts):
    return tuple(None if t is None else t.cuda() for t in ts)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "rows,d_model,hidden,blocks,bias,activation",
    [
        (1000, 128, 64, 8, False, "relu"),  # benchmark configuration 2 at a size the oracle finishes quickly
        (300, 128, 64, 2, True, "relu"),
        (257, 64, 32, 3, True, "silu"),
        (129, 32, 16, 1, False, "none"),
        (128, 96, 48, 2, True, "relu2"),
        (5, 128, 64, 8, True, "relu"),
    ],
)
def test_forward_backward_against_oracle(dtype, rows, d_model, hidden, blocks, bias, activation):
    weights, biases = make_params(blocks, d_model // 2, hidden, bias, dtype, seed=rows)
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, d_model, generator=g).to(dtype)
    go = torch.randn(rows, d_model, generator=g).to(dtype)
    y_r, dx_r, grads_r, xrec_r = oracle.forward_backward_storage_rounded(x, weights, biases, go, activation)
    y32 = oracle.forward(x, *weights, *biases, activation=activation)

    wc, bc = to_cuda(weights), to_cuda(biases)
    y = reversible_mlp_forward(x.cuda(), wc, bc, activation)
    assert y.shape == x.shape and y.dtype == dtype
    assert nerr(y, y32) <= LOOSE[dtype], f"y vs float32: {nerr(y, y32)}"
    assert rows_outside(y, y_r, TIGHT[dtype]) <= 1e-2

    got = reversible_mlp_backward(y, go.cuda(), wc, bc, activation, reconstruct=True)
    # the backward pass is checked from the y it was given, so forward differences do not leak in
    _, dx_r, grads_r, xrec_r = oracle.forward_backward_storage_rounded(x, weights, biases, go, activation, y_saved=y.cpu())
    # rows where a ReLU sits within rounding noise of zero may switch differently: allow a few
    assert rows_outside(got.dx, dx_r, 2 * TIGHT[dtype]) <= 5e-2, rows_outside(got.dx, dx_r, 2 * TIGHT[dtype])
    assert rows_outside(got.x_reconstructed, xrec_r, 2 * TIGHT[dtype]) <= 5e-2
    for name, want, have in zip(("dw_f1", "dw_f2", "dw_g1", "dw_g2", "db_f1", "db_f2", "db_g1", "db_g2"), grads_r, got[1:9]):
        assert (want is None) == (have is None), name
        if want is not None:
            # The block undone first (the last one) sees no accumulated divergence: tight.  Earlier
            # blocks inherit the few rows whose ReLUs switched on a one-ulp difference upstream.
            per_block = want.shape[0] // blocks
            assert nerr(have[-per_block:], want[-per_block:]) <= 5 * TIGHT[dtype], f"{name} (last block): {nerr(have[-per_block:], want[-per_block:])}"
            assert nerr(have, want) <= (5 * TIGHT[dtype] if blocks <= 3 else 0.15), f"{name}: {nerr(have, want)}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1024, 1300])
def test_every_block_is_tight_without_an_activation(dtype, rows):
    # Benchmark configuration 2's stack (8 blocks, d_model 128, hidden 64, no biases) with activation "none":
    # no ReLU can switch on a one-ulp difference, so EVERY block's weight gradient - not only the last one's -
    # must sit within the tight tolerance of the oracle that rounds where the kernels round.  A kernel that
    # mis-addressed one block's gradient flush, or mixed up two blocks' weights, fails here by orders of magnitude.
    d_model, hidden, blocks = 128, 64, 8
    weights, biases = make_params(blocks, d_model // 2, hidden, False, dtype, seed=11)
    weights = tuple((w.float() * 0.5).to(dtype) for w in weights)  # keep the linear stack's activations of order one
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, d_model, generator=g).to(dtype)
    go = torch.randn(rows, d_model, generator=g).to(dtype)
    wc = to_cuda(weights)
    y = reversible_mlp_forward(x.cuda(), wc, (None,) * 4, "none")
    y_r, _, _, _ = oracle.forward_backward_storage_rounded(x, weights, biases, go, "none")
    assert nerr(y, y_r) <= 2 * TIGHT[dtype]
    got = reversible_mlp_backward(y, go.cuda(), wc, (None,) * 4, "none", reconstruct=True)
    _, dx_r, grads_r, xrec_r = oracle.forward_backward_storage_rounded(x, weights, biases, go, "none", y_saved=y.cpu())
    assert nerr(got.dx, dx_r) <= 5 * TIGHT[dtype], nerr(got.dx, dx_r)
    assert nerr(got.x_reconstructed, xrec_r) <= 5 * TIGHT[dtype]
    for name, want, have in zip(("dw_f1", "dw_f2", "dw_g1", "dw_g2"), grads_r[:4], got[1:5]):
        per_block = want.shape[0] // blocks
        for b in range(blocks):
            err = nerr(have[b * per_block : (b + 1) * per_block], want[b * per_block : (b + 1) * per_block])
            assert err <= 5 * TIGHT[dtype], f"{name}, block {b}: {err}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_autograd_function_against_float32_autograd(dtype):
    # through the autograd.Function, against torch autograd with stored activations (float32)
    rows, d_model, hidden, blocks = 4096, 128, 64, 8
    weights, biases = make_params(blocks, d_model // 2, hidden, False, dtype, seed=3)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, rows // 4, d_model, generator=g).to(dtype)
    go = torch.randn(4, rows // 4, d_model, generator=g).to(dtype)
    y32, dx32, grads32 = oracle.forward_backward(x, weights, biases, go)

    leaves = [w.cuda().requires_grad_(True) for w in weights]
    xc = x.cuda().requires_grad_(True)
    y = reversible_mlp(xc, *leaves)
    assert y.shape == x.shape
    y.backward(go.cuda())
    _, dx_r, grads_r, _ = oracle.forward_backward_storage_rounded(x, weights, biases, go, y_saved=y.detach().cpu())
    assert nerr(y, y32) <= LOOSE[dtype]
    # gradients: the north-star tolerance, or 1.5x the distance between the float32 oracle and the
    # oracle that rounds where 16-bit kernels must round (ReLU switches near zero), whichever is larger
    assert rows_outside(xc.grad, dx32, LOOSE[dtype]) <= max(1e-2, 1.5 * rows_outside(dx_r, dx32, LOOSE[dtype]))
    for w, want, want_r in zip(leaves, grads32[:4], grads_r[:4]):
        assert nerr(w.grad, want) <= max(LOOSE[dtype], 1.5 * nerr(want_r, want)), (nerr(w.grad, want), nerr(want_r, want))
        per_block = want.shape[0] // blocks
        assert nerr(w.grad[-per_block:], want_r[-per_block:]) <= 5 * TIGHT[dtype], nerr(w.grad[-per_block:], want_r[-per_block:])


def test_reconstruction_at_full_baseline_size():
    # bf16 [2^20, 128], 8 blocks of 64 -> 64 -> 64: the backward pass recovers the input it never saw
    rows, d_model, hidden, blocks = 2**20, 128, 64, 8
    dtype = torch.bfloat16
    weights, _ = make_params(blocks, d_model // 2, hidden, False, dtype, seed=5)
    wc = to_cuda(weights)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(rows, d_model, device="cuda", generator=g).to(dtype)
    go = torch.randn(rows, d_model, device="cuda", generator=g).to(dtype)
    y = reversible_mlp_forward(x, wc, (None,) * 4)
    got = reversible_mlp_backward(y, go, wc, (None,) * 4, reconstruct=True)
    err = (got.x_reconstructed.float() - x.float()).abs()
    scale = float(x.float().abs().max())
    # one bf16 rounding of the output, carried back through 8 blocks
    assert float(err.max()) / scale <= 5e-2 and float(err.mean()) / scale <= 2e-3
    # linearity of the backward pass in grad_out (the weight gradients are sums over all rows)
    got2 = reversible_mlp_backward(y, go * 2, wc, (None,) * 4)
    assert nerr(got2.dw_f1.float(), got.dw_f1.float() * 2) <= 2e-2
    assert torch.isfinite(got.dx.float()).all()


def test_empty_batch_leading_dims_and_checks():
    dtype = torch.float16
    weights, biases = make_params(2, 64, 64, True, dtype)
    wc, bc = to_cuda(weights), to_cuda(biases)
    assert reversible_mlp(torch.empty(0, 128, device="cuda", dtype=dtype), *wc, *bc).shape == (0, 128)
    x = torch.randn(3, 7, 128, device="cuda").to(dtype)
    y = reversible_mlp(x, *wc, *bc)
    want = oracle.forward(x.cpu(), *weights, *biases)
    assert y.shape == (3, 7, 128) and nerr(y, want) <= 1e-2
    with pytest.raises(AssertionError, match="Invalid activation"):
        reversible_mlp(x, *wc, *bc, activation="gelu")
    with pytest.raises(AssertionError, match="every layer or for none"):
        reversible_mlp(x, *wc, bc[0], None, None, None)
    with pytest.raises(AssertionError, match="weight shape mismatch"):
        reversible_mlp(x[..., :64], *wc, *bc)
    with pytest.raises(TypeError):
        reversible_mlp(x.float(), *(w.float() for w in wc))


def test_module_under_autocast():
    torch.manual_seed(0)
    layer = ReversibleMLP(d_model=128, blocks=4, d_hidden=64, bias=True).cuda()
    assert set(layer.state_dict().keys()) == {f"{k}_{n}" for k in ("w", "b") for n in ("f1", "f2", "g1", "g2")}
    x = torch.randn(2, 50, 128, device="cuda", requires_grad=True)
    with torch.autocast(device_type="cuda", dtype=torch.float16):
        y = layer(x)
    assert y.dtype == torch.float16
    y.float().pow(2).sum().backward()
    params = [layer.w_f1, layer.w_f2, layer.w_g1, layer.w_g2, layer.b_f1, layer.b_f2, layer.b_g1, layer.b_g2]
    assert all(p.grad is not None and p.grad.dtype == torch.float32 for p in params)
    cpu = [p.detach().cpu() for p in params]
    xr = x.detach().cpu().half()
    yo = oracle.forward(xr, *[c.half() for c in cpu])
    assert nerr(y, yo) <= 1e-2
    w16, b16 = [c.half() for c in cpu[:4]], [c.half() for c in cpu[4:]]
    _, _, grads32 = oracle.forward_backward(xr, w16, b16, 2 * yo)
    _, _, grads_r, _ = oracle.forward_backward_storage_rounded(xr, w16, b16, 2 * yo)
    assert nerr(layer.w_f1.grad, grads32[0]) <= max(1e-2, 1.5 * nerr(grads_r[0], grads32[0]))
    assert x.grad is not None and x.grad.shape == x.shape


def test_tensor_core_kernels_never_timed_out():
    from triton_helpers_b200 import _lib

    assert _lib.lib().th_rev_tc_status() == 0


def test_mma_sync_kernels_still_pass_when_selected():
    # TH_MLP_LEGACY=1 routes every call to the mma.sync kernels (which also serve biased and SiLU /
    # ReLU^2 backward passes); rerun the oracle comparisons that way in a fresh process
    import os
    import subprocess
    import sys

    if os.environ.get("TH_MLP_LEGACY") == "1":
        pytest.skip("already running on the mma.sync kernels")
    env = dict(os.environ, TH_MLP_LEGACY="1")
    cmd = [sys.executable, "-m", "pytest", __file__, "-q", "-x", "-m", "gpu", "-k", "against_oracle or float32_autograd"]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-2000:]


def test_forward_through_shared_memory_still_passes_when_selected():
    # TH_MLP_NO_TMEM_A=1 keeps the forward kernel's A operands in shared-memory operand tiles instead of tensor memory
    import os
    import subprocess
    import sys

    if os.environ.get("TH_MLP_NO_TMEM_A") == "1" or os.environ.get("TH_MLP_LEGACY") == "1":
        pytest.skip("already running without the tensor-memory A operand")
    env = dict(os.environ, TH_MLP_NO_TMEM_A="1")
    cmd = [sys.executable, "-m", "pytest", __file__, "-q", "-x", "-m", "gpu", "-k", "against_oracle or float32_autograd"]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-2000:]
