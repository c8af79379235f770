r"""CPU checks of the MLP oracles: the storage-rounded restatements collapse to plain float32
autograd when the storage dtype is float32, and the reversible stack inverts exactly."""
import pytest
import torch

from oracle import fused_mlp, reversible_mlp


def _rev_params(blocks, half, hidden, bias, dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed)
    u = lambda *shape, fan: ((torch.rand(*shape, generator=g) * 2 - 1) / fan**0.5).to(dtype)  # noqa: E731
    weights = (u(blocks * hidden, half, fan=half), u(blocks * half, hidden, fan=hidden),
               u(blocks * hidden, half, fan=half), u(blocks * half, hidden, fan=hidden))  # fmt: skip
    biases = (u(blocks, hidden, fan=half), u(blocks, half, fan=hidden), u(blocks, hidden, fan=half),
              u(blocks, half, fan=hidden)) if bias else (None,) * 4  # fmt: skip
    return weights, biases


@pytest.mark.parametrize("activation", ["relu", "silu", "relu2", "none"])
def test_fused_mlp_rounded_oracle_equals_autograd_in_float32(activation):
    torch.manual_seed(0)
    lin = [torch.nn.Linear(8, 16), torch.nn.Linear(16, 16), torch.nn.Linear(16, 16), torch.nn.Linear(16, 4)]
    w_hid = torch.cat([lin[1].weight, lin[2].weight]).detach()
    b_hid = torch.stack([lin[1].bias, lin[2].bias]).detach()
    args = (lin[0].weight.detach(), lin[0].bias.detach(), lin[3].weight.detach(), lin[3].bias.detach(), w_hid, b_hid)
    x, go = torch.randn(2, 5, 8), torch.randn(2, 5, 4)
    a = fused_mlp.forward_backward(x, *args, go, activation)
    b = fused_mlp.forward_backward_storage_rounded(x, *args, go, activation)
    for u, v in zip(a, b):
        torch.testing.assert_close(u, v, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("activation", ["relu", "silu"])
def test_reversible_rounded_oracle_equals_autograd_in_float32(bias, activation):
    weights, biases = _rev_params(3, 16, 32, bias)
    g = torch.Generator().manual_seed(1)
    x, go = torch.randn(7, 32, generator=g), torch.randn(7, 32, generator=g)
    y, dx, grads = reversible_mlp.forward_backward(x, weights, biases, go, activation)
    y2, dx2, grads2, x_rec = reversible_mlp.forward_backward_storage_rounded(x, weights, biases, go, activation)
    torch.testing.assert_close(y, y2, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(dx, dx2, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(x_rec, x, rtol=1e-4, atol=1e-5)
    for u, v in zip(grads, grads2):
        assert (u is None) == (v is None)
        if u is not None:
            torch.testing.assert_close(u, v, rtol=1e-4, atol=1e-5)


def test_reversible_reconstruct_inverts_forward():
    weights, biases = _rev_params(8, 64, 64, True)
    x = torch.randn(50, 128, generator=torch.Generator().manual_seed(2))
    y = reversible_mlp.forward(x, *weights, *biases)
    torch.testing.assert_close(reversible_mlp.reconstruct(y, *weights, *biases), x, rtol=1e-4, atol=1e-4)


def test_fused_mlp_oracle_is_a_linear_chain():
    # depth 1 (no hidden stack), no bias, no activation: y = x W_in^T W_out^T
    g = torch.Generator().manual_seed(3)
    x, w_in, w_out = torch.randn(1, 9, 5, generator=g), torch.randn(16, 5, generator=g), torch.randn(3, 16, generator=g)
    want = x @ w_in.t() @ w_out.t()
    torch.testing.assert_close(fused_mlp.forward(x, w_in, None, w_out, None, activation="none"), want)
