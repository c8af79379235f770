r"""The kernels that fuse the hash encoding with the MLP (``th_field_fwd`` / ``th_field_bwd``) against the
CPU oracles and against the separate CUDA operators they stand for."""
import pytest
import torch

from oracle import fused_mlp as mlp_oracle
from oracle import hash_encoding as hash_oracle
from triton_helpers_b200 import _lib
from triton_helpers_b200.layers.fully_fused_mlp import FullyFusedMLP, fully_fused_mlp
from triton_helpers_b200.layers.hash_encoding import HashEncoding, hash_encoding
from triton_helpers_b200.layers.hash_encoding.helpers import level_geometry
from triton_helpers_b200.layers.hash_encoding.kernel import _default_pi, _Launch
from triton_helpers_b200.layers.neural_field import field_backward, field_forward, hash_encoded_mlp
from triton_helpers_b200.layers.neural_field.kernel import FieldUnsupported
from triton_helpers_b200.training import NeuralFieldTrainer

pytestmark = pytest.mark.gpu


def nerr(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def make_case(n, D, F, T, L, lo, hi, d_hidden, d_out, depth, dtype, seed=0, clustered=False):
    g = torch.Generator().manual_seed(seed)
    geo = level_geometry(L, T, D, lo, hi)
    x = torch.rand(n, D, generator=g)
    if clustered:
        x = (0.5 + 0.01 * torch.randn(n, D, generator=g)).clamp_(0, 1 - 2**-24)
    table = (torch.rand(geo.total_rows, F, generator=g) * 2 - 1).to(dtype)
    lin = lambda o, i: ((torch.rand(o, i, generator=g) * 2 - 1) / i**0.5).to(dtype)  # noqa: E731
    d_in = L * F
    w_in, w_out = lin(d_hidden, d_in), lin(d_out, d_hidden)
    w_hid = torch.cat([lin(d_hidden, d_hidden) for _ in range(depth - 1)], 0) if depth > 1 else None
    go = (torch.randn(n, d_out, generator=g) * 0.1).to(dtype)
    return dict(x=x, table=table, w_in=w_in, w_out=w_out, w_hid=w_hid, go=go, geo=geo, kw=dict(table_cap=T, levels=L, n_min=lo, n_max=hi))


CASES = [
    # n, D, F, T, L, lo, hi, d_hidden, d_out, depth, dtype, activation
    (1, 3, 2, 2**14, 16, 16, 512, 64, 16, 2, torch.float16, "relu"),
    (127, 3, 2, 2**14, 16, 16, 512, 64, 16, 2, torch.float16, "relu"),
    (129, 3, 2, 2**14, 8, 16, 256, 32, 8, 1, torch.float16, "relu"),
    (4099, 3, 2, 2**19, 16, 16, 2048, 64, 16, 2, torch.float16, "relu"),
    (4099, 3, 2, 2**14, 16, 16, 512, 64, 16, 4, torch.bfloat16, "relu"),
    (5000, 2, 4, 2**12, 8, 8, 256, 64, 24, 2, torch.float16, "none"),
    (5000, 3, 4, 2**14, 16, 16, 512, 64, 16, 3, torch.bfloat16, "relu"),
    (5000, 2, 2, 2**10, 16, 4, 512, 16, 5, 2, torch.float16, "relu"),
    (70001, 3, 2, 2**14, 16, 16, 512, 64, 16, 2, torch.float16, "relu"),  # large enough for the shared-memory coarse levels
]


def _launch(c, dev, L, T, lo, hi, scale=1.0):
    x = c["x"].to(dev)
    return _Launch(x, _default_pi(dev), x.shape[1], T, L, lo, hi, scale), x


@pytest.mark.parametrize("n,D,F,T,L,lo,hi,d_hidden,d_out,depth,dtype,activation", CASES)
def test_fused_forward_matches_oracle_and_the_separate_operators(n, D, F, T, L, lo, hi, d_hidden, d_out, depth, dtype, activation):
    dev = torch.device("cuda")
    c = make_case(n, D, F, T, L, lo, hi, d_hidden, d_out, depth, dtype)
    launch, x = _launch(c, dev, L, T, lo, hi)
    table, w_in, w_out = c["table"].to(dev), c["w_in"].to(dev), c["w_out"].to(dev)
    w_hid = None if c["w_hid"] is None else c["w_hid"].to(dev)
    feats = torch.full((n, L * F), float("nan"), device=dev, dtype=dtype)
    out = torch.full((n, d_out), float("nan"), device=dev, dtype=dtype)
    field_forward(launch, table, w_in, w_out, w_hid, activation, L, feats_out=feats, out=out)
    # the encoding written for the backward pass is exactly the stand-alone encoding
    want_feats = hash_encoding(x, table, None, None, T, lo, hi, L)
    assert torch.equal(feats, want_feats)
    # oracle: encoding (rounded to the table dtype like the operand tile) -> float32 MLP
    enc = hash_oracle.encode(c["x"], c["table"], **c["kw"])
    want = mlp_oracle.forward(enc.unsqueeze(0), c["w_in"], None, c["w_out"], None, c["w_hid"], None, activation=activation).squeeze(0)
    assert nerr(out, want) <= 1e-2
    # the separate CUDA operators on the same values
    sep = fully_fused_mlp(want_feats.unsqueeze(0), w_in, None, w_out, None, w_hid, None, activation).squeeze(0)
    assert nerr(out, sep) <= 2e-3
    assert _lib.lib().th_mlp_tc_status() == 0


@pytest.mark.parametrize("n,D,F,T,L,lo,hi,d_hidden,d_out,depth,dtype,activation", [c for c in CASES if c[8] % 8 == 0])
def test_fused_forward_with_loss(n, D, F, T, L, lo, hi, d_hidden, d_out, depth, dtype, activation):
    dev = torch.device("cuda")
    c = make_case(n, D, F, T, L, lo, hi, d_hidden, d_out, depth, dtype, seed=1)
    launch, x = _launch(c, dev, L, T, lo, hi)
    table, w_in, w_out = c["table"].to(dev), c["w_in"].to(dev), c["w_out"].to(dev)
    w_hid = None if c["w_hid"] is None else c["w_hid"].to(dev)
    target = torch.rand(n, d_out, device=dev).to(dtype)
    out = torch.empty(n, d_out, device=dev, dtype=dtype)
    grad = torch.empty(n, d_out, device=dev, dtype=dtype)
    loss = torch.zeros(1, device=dev)
    field_forward(launch, table, w_in, w_out, w_hid, activation, L, out=out, target=target, grad_out=grad, loss_sum=loss, grad_scale=0.25)
    diff = out.float() - target.float()
    assert torch.equal(grad, (diff * 0.25).to(dtype))
    torch.testing.assert_close(loss[0], (diff * diff).sum(), rtol=1e-4, atol=1e-6)
    # without the prediction output
    grad2, loss2 = torch.empty_like(grad), torch.zeros(1, device=dev)
    field_forward(launch, table, w_in, w_out, w_hid, activation, L, target=target, grad_out=grad2, loss_sum=loss2, grad_scale=0.25)
    assert torch.equal(grad, grad2)


@pytest.mark.parametrize("n,D,F,T,L,lo,hi,d_hidden,d_out,depth,dtype,activation", CASES)
def test_fused_backward_matches_oracle_and_the_separate_operators(n, D, F, T, L, lo, hi, d_hidden, d_out, depth, dtype, activation):
    dev = torch.device("cuda")
    c = make_case(n, D, F, T, L, lo, hi, d_hidden, d_out, depth, dtype, seed=2)
    launch, x = _launch(c, dev, L, T, lo, hi)
    table = c["table"].to(dev)
    weights = [None if w is None else w.to(dev).requires_grad_(True) for w in (c["w_in"], c["w_out"], c["w_hid"])]
    go = c["go"].to(dev)
    feats = hash_encoding(x, table, None, None, T, lo, hi, L)
    # fused
    grad_table = torch.zeros_like(table)
    grad_feats = torch.empty_like(feats)
    lib = _lib.lib()
    ws = torch.empty(lib.th_field_workspace_bytes(L, F, d_hidden, d_out, depth) // 4, device=dev)
    field_backward(launch, feats, go, weights[0].detach(), weights[1].detach(), None if weights[2] is None else weights[2].detach(),
                   activation, L, grad_table, ws, grad_feats=grad_feats)
    assert lib.th_mlp_tc_status() == 0 and lib.th_hash_status() == 0
    # separate CUDA operators: MLP backward, then encoding backward of its feature gradient
    f = feats.detach().clone().requires_grad_(True)
    y = fully_fused_mlp(f.unsqueeze(0), weights[0], None, weights[1], None, weights[2], None, activation)
    y.backward(go.unsqueeze(0))
    assert torch.equal(grad_feats, f.grad)  # same MMAs on the same operands, same rounding
    t = table.detach().clone().requires_grad_(True)
    hash_encoding(x, t, None, None, T, lo, hi, L).backward(f.grad)
    assert nerr(grad_table, t.grad) <= 2e-2  # 16-bit reductions in varying order
    sizes = [weights[0].numel(), 0 if weights[2] is None else weights[2].numel(), weights[1].numel()]
    got = torch.split(ws[: sum(sizes)], sizes)
    for sums, w in ((got[0], weights[0]), (got[2], weights[1])) + (() if weights[2] is None else ((got[1], weights[2]),)):
        assert nerr(sums.view_as(w), w.grad.float()) <= 4e-3  # the separate operator rounds its float32 sums to 16 bits
    # oracle: float32 table gradient of the rounded feature gradient (no 16-bit accumulation)
    want_table = hash_oracle.encode_backward(c["x"], grad_feats.float().cpu(), c["table"].float(), **c["kw"])
    assert nerr(grad_table, want_table) <= 2e-2
    ref = mlp_oracle.forward_backward_storage_rounded(feats.cpu().unsqueeze(0), c["w_in"], None, c["w_out"], None, c["w_hid"], None,
                                                      c["go"].float().unsqueeze(0), activation=activation)
    assert nerr(got[0].view_as(weights[0]), ref[2]) <= 1e-2
    assert nerr(got[2].view_as(weights[1]), ref[4]) <= 1e-2


def test_fused_backward_clustered_points_hit_the_same_cells():
    # every point inside a few cells of the coarse levels: warp aggregation and the shared-memory copy at work
    n, D, F, T, L, lo, hi = 2**17, 3, 2, 2**14, 16, 16, 512
    dev = torch.device("cuda")
    c = make_case(n, D, F, T, L, lo, hi, 64, 16, 2, torch.float16, seed=5, clustered=True)
    launch, x = _launch(c, dev, L, T, lo, hi)
    table = c["table"].to(dev)
    w_in, w_out, w_hid = c["w_in"].to(dev), c["w_out"].to(dev), c["w_hid"].to(dev)
    go = (c["go"].float() * 0.01).half().to(dev)
    feats = hash_encoding(x, table, None, None, T, lo, hi, L)
    grad_table, grad_feats = torch.zeros_like(table), torch.empty_like(feats)
    ws = torch.empty(_lib.lib().th_field_workspace_bytes(L, F, 64, 16, 2) // 4, device=dev)
    field_backward(launch, feats, go, w_in, w_out, w_hid, "relu", L, grad_table, ws, grad_feats=grad_feats)
    want = hash_oracle.encode_backward(c["x"], grad_feats.float().cpu(), c["table"].float(), **c["kw"])
    assert nerr(grad_table, want) <= 3e-2
    assert _lib.lib().th_hash_status() == 0


def test_hash_encoded_mlp_autograd_equals_the_two_layers():
    dev = torch.device("cuda")
    torch.manual_seed(0)
    enc = HashEncoding(2**14, 16, 3, 2, 16, 512).to(dev).half()
    mlp = FullyFusedMLP(32, 64, 16, depth=3, bias=False).to(dev).half()
    x = torch.rand(3, 1000, 3, device=dev)
    go = torch.randn(3, 1000, 16, device=dev).half() * 0.1
    want = mlp(enc(x).view(1, -1, 32)).view(3, 1000, 16)
    want.backward(go)
    grads = {n: p.grad.clone() for n, p in list(enc.named_parameters()) + list(mlp.named_parameters())}
    for p in list(enc.parameters()) + list(mlp.parameters()):
        p.grad = None
    got = hash_encoded_mlp(x, enc.embeddings, mlp.w_in, mlp.w_out, mlp.w_hid, enc.pi, 2**14, 16, 512, 16, "relu")
    assert got.shape == want.shape and nerr(got, want) <= 2e-3
    got.backward(go)
    assert nerr(enc.embeddings.grad, grads["embeddings"]) <= 2e-2
    for name in ("w_in", "w_hid", "w_out"):
        assert nerr(getattr(mlp, name).grad, grads[name]) <= 4e-3, name
    # no gradient wanted: the encoding is not written out at all
    with torch.no_grad():
        again = hash_encoded_mlp(x, enc.embeddings, mlp.w_in, mlp.w_out, mlp.w_hid, enc.pi, 2**14, 16, 512, 16, "relu")
    assert torch.equal(again, got)


def test_unsupported_configurations_are_refused_not_miscomputed():
    dev = torch.device("cuda")
    x = torch.rand(100, 3, device=dev)
    table = torch.randn(level_geometry(16, 2**14, 3, 16, 512).total_rows, 2, device=dev)  # float32 table
    w_in, w_out = torch.randn(64, 32, device=dev), torch.randn(16, 64, device=dev)
    with pytest.raises(FieldUnsupported):
        hash_encoded_mlp(x, table, w_in, w_out, None, None, 2**14, 16, 512, 16, "relu")
    with pytest.raises(FieldUnsupported):  # SiLU needs the pre-activation in backward: not built into the fused kernels
        hash_encoded_mlp(x, table.half(), w_in.half(), w_out.half(), None, None, 2**14, 16, 512, 16, "silu")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_trainer_fused_and_separate_paths_see_the_same_gradients(dtype):
    g = torch.Generator().manual_seed(4)
    coords = torch.rand(20000, 3, generator=g).cuda()
    targets = torch.rand(20000, 8, generator=g).cuda().to(dtype)

    def moments(fused):
        torch.manual_seed(3)
        enc = HashEncoding(2**12, 8, 3, 2, 8, 128)
        mlp = FullyFusedMLP(16, 32, 8, depth=2, bias=False)
        trainer = NeuralFieldTrainer(enc.cuda().to(dtype), mlp.cuda().to(dtype), lr=0.0, betas=(0.0, 0.0), grad_out_scale=0.25, fused=fused)
        loss = float(trainer.step(coords, targets))
        return loss, trainer._state.table_m.clone(), trainer._state.mlp_m.clone()

    loss_b, table_b, mlp_b = moments(False)
    for mode in (True, "backward", None):
        loss_a, table_a, mlp_a = moments(mode)
        assert abs(loss_a - loss_b) <= 1e-4 * abs(loss_b)
        # table gradients are summed with 16-bit reductions in varying order: 11 significant bits in float16, 8 in bfloat16
        assert nerr(table_a, table_b) <= (2e-2 if dtype == torch.float16 else 8e-2) and nerr(mlp_a, mlp_b) <= 5e-3
