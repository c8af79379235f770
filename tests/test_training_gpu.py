r"""The training-step glue on the GPU: MSE-gradient kernel, Adam kernel, and the whole
hash-encoding -> fused-MLP step against the CPU port (``oracle/training_step.py``)."""
import pytest
import torch

from oracle.training_step import CpuNeuralField, make_batch
from triton_helpers_b200 import _lib
from triton_helpers_b200.layers.fully_fused_mlp import FullyFusedMLP
from triton_helpers_b200.layers.hash_encoding import HashEncoding
from triton_helpers_b200.optim import FusedAdam
from triton_helpers_b200.training import NeuralFieldTrainer, mse_grad

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n", [0, 7, 4096, 100003])
def test_mse_grad_kernel(dtype, n):
    g = torch.Generator(device="cuda").manual_seed(n)
    pred = torch.randn(n, device="cuda", generator=g).to(dtype)
    target = torch.rand(n, device="cuda", generator=g).to(dtype)
    grad, loss_sum = mse_grad(pred, target, 0.25)
    diff = pred.float() - target.float()
    assert grad.dtype == dtype and grad.shape == pred.shape
    torch.testing.assert_close(grad.float(), (diff * 0.25).to(dtype).float(), rtol=0, atol=0)
    torch.testing.assert_close(loss_sum[0], (diff * diff).sum(), rtol=1e-4, atol=1e-6)


def test_adam_kernel_matches_torch_adam_in_float32():
    g = torch.Generator(device="cuda").manual_seed(0)
    shapes = [(1000, 2), (64, 32), (13,)]
    ours = [torch.randn(*s, device="cuda", generator=g).requires_grad_(True) for s in shapes]
    ref = [p.detach().clone().requires_grad_(True) for p in ours]
    opt = FusedAdam(ours, lr=1e-2, betas=(0.9, 0.99), eps=1e-15)
    opt_ref = torch.optim.Adam(ref, lr=1e-2, betas=(0.9, 0.99), eps=1e-15)
    for step in range(5):
        for p, q in zip(ours, ref):
            grad = torch.randn(p.shape, device="cuda", generator=g) * 10.0 ** (step - 3)
            p.grad, q.grad = grad.clone(), grad.clone()
        opt.step()
        opt_ref.step()
        for p, q in zip(ours, ref):
            torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-7)


def test_adam_kernel_half_parameters_grad_scale_and_zero_grad():
    g = torch.Generator(device="cuda").manual_seed(1)
    master = torch.randn(5001, 2, device="cuda", generator=g) * 1e-2
    p16 = master.half().requires_grad_(True)
    p32 = master.half().float().requires_grad_(True)
    opt16 = FusedAdam([p16], lr=1e-2, betas=(0.9, 0.99), eps=1e-15)
    opt32 = torch.optim.Adam([p32], lr=1e-2, betas=(0.9, 0.99), eps=1e-15)
    for _ in range(3):
        true_grad = torch.randn(master.shape, device="cuda", generator=g) * 1e-5  # g*g underflows float16
        p16.grad = (true_grad * 1024).half()  # stored with a loss scale of 1024
        p32.grad = p16.grad.float() / 1024
        opt16.step(grad_scale=1.0 / 1024, zero_grad=True)
        opt32.step()
        assert float(p16.grad.abs().max()) == 0.0  # cleared in the same pass
        # float32 moments: the update matches float32 Adam up to the rounding of the stored parameter
        torch.testing.assert_close(p16.float(), p32.half().float(), rtol=2e-3, atol=1e-6)
        p32.data.copy_(p16.float())  # keep the two trajectories on the same (rounded) parameters


def test_training_step_tracks_the_cpu_port():
    # same initial parameters and batch as the CPU port; float16 table and MLP on the GPU
    kw = dict(levels=8, table_cap=2**12, n_min=16, n_max=256, d_hidden=64, d_out=16, depth=2, seed=0)
    cpu = CpuNeuralField(**kw)
    enc = HashEncoding(kw["table_cap"], kw["levels"], 3, 2, kw["n_min"], kw["n_max"])
    mlp = FullyFusedMLP(kw["levels"] * 2, 64, 16, depth=2, bias=False)
    with torch.no_grad():
        enc.embeddings.copy_(cpu.params["table"])
        mlp.w_in.copy_(cpu.params["w_in"])
        mlp.w_hid.copy_(cpu.params["w_hid"])
        mlp.w_out.copy_(cpu.params["w_out"])
    trainer = NeuralFieldTrainer(enc.cuda().half(), mlp.cuda().half(), lr=1e-2, betas=(0.9, 0.99), eps=1e-15)
    coords, targets = make_batch(8192, d_out=16, seed=3)
    gpu_losses, cpu_losses = [], []
    for _ in range(6):
        gpu_losses.append(float(trainer.step(coords.cuda(), targets.cuda().half())))
        cpu_losses.append(cpu.step(coords, targets))
    # the table part of the flat gradient buffer was cleared by the Adam pass that consumed it
    assert float(trainer.encoding.embeddings.grad.abs().max()) == 0.0
    assert trainer.skipped_elements() == 0
    assert gpu_losses[-1] < gpu_losses[0]
    for a, b in zip(gpu_losses, cpu_losses):
        assert abs(a - b) <= 2e-2 * abs(b), (gpu_losses, cpu_losses)
    # the prediction path alone (no optimisation) agrees with the CPU port to float16 accuracy
    fresh = CpuNeuralField(**kw)
    with torch.no_grad():
        for name, dst in (("table", enc.embeddings), ("w_in", mlp.w_in), ("w_hid", mlp.w_hid), ("w_out", mlp.w_out)):
            dst.copy_(fresh.params[name].to(dst.device, dst.dtype))
        got = trainer(coords.cuda())
        want = fresh.predict(coords)
    assert float((got.float().cpu() - want).abs().max() / want.abs().max()) <= 1e-2


def _small_trainer(backward_passes=None, dtype=torch.float16, bias=False, seed=3):
    torch.manual_seed(seed)
    enc = HashEncoding(2**12, 8, 3, 2, 8, 128)
    mlp = FullyFusedMLP(16, 32, 8, depth=2, bias=bias)
    return NeuralFieldTrainer(enc.cuda().to(dtype), mlp.cuda().to(dtype), lr=1e-2, backward_passes=backward_passes)


@pytest.mark.parametrize("bias", [False, True])
def test_direct_step_matches_the_layers_autograd(bias):
    # The direct step (C ABI on persistent buffers, normalised MLP gradients in the flat buffer) sees the
    # same gradient of mean((pred - target)^2) as forward + backward through the two autograd functions.
    # With beta1 = 0 Adam's first moment after one step IS the gradient it was given (stored gradient x
    # its scale), which is what the two paths are compared on; lr = 0 keeps the parameters.
    g = torch.Generator().manual_seed(4)
    coords = torch.rand(8192, 3, generator=g).cuda()
    targets = torch.rand(8192, 8, generator=g).cuda().half()
    scale = 1.0 / 4
    ref = _small_trainer(bias=bias)
    pred = ref(coords)
    grad_out, loss_sum = mse_grad(pred, targets, scale)
    pred.backward(grad_out)
    true = {n: p.grad.float() * (2.0 / (pred.numel() * scale)) for n, p in ref.named_parameters()}

    direct = _small_trainer(bias=bias)
    direct.grad_out_scale, direct.lr, direct.betas = scale, 0.0, (0.0, 0.0)
    loss = direct.step(coords, targets)
    assert abs(float(loss) - float(loss_sum) / pred.numel()) <= 1e-3 * float(loss)
    st = direct._state
    got = {"encoding.embeddings": st.table_m.view_as(direct.encoding.embeddings)}
    offset = 0
    for name in ("w_in", "w_hid", "w_out") + (("b_in", "b_hid", "b_out") if bias else ()):
        p = getattr(direct.mlp, name)
        got["mlp." + name] = st.mlp_m[offset : offset + p.numel()].view_as(p)
        offset += p.numel()
    # the flat MLP buffers follow th_mlp_bwd's workspace layout, which reserves the bias slots also for a bias-free network
    assert offset <= st.mlp_m.numel() and float(st.mlp_m[offset:].abs().sum()) == 0.0 and set(got) == set(true)
    for name, want in true.items():
        err = float((got[name] - want).abs().max() / want.abs().max())
        assert err <= 2e-2, f"{name}: {err}"  # float16 storage of the gradients, reductions in varying order
    assert direct.skipped_elements() == 0
    # and the parameters are the same objects the layers use: a real step moves the MLP's prediction
    direct.lr = 1e-2
    before = direct(coords).float()
    direct.step(coords, targets)
    assert float((direct(coords).float() - before).abs().max()) > 0


def test_backward_in_level_passes_matches_the_single_pass():
    # the backward a multi-rank run may take (encoding backward range by range, sums started in
    # between), here on one rank where the sums are no-ops: same gradients as the single-pass backward
    g = torch.Generator().manual_seed(4)
    coords = torch.rand(8192, 3, generator=g).cuda()
    targets = torch.rand(8192, 8, generator=g).cuda().half()

    def grads(passes):
        trainer = _small_trainer(passes)
        trainer.lr = 0.0  # keep the parameters; Adam still clears the table gradient, so look at its first moment
        trainer.betas = (0.0, 0.0)
        loss = float(trainer.step(coords, targets))
        st = trainer._state
        return loss, {"table": st.table_m.clone(), "mlp": st.mlp_m.clone()}

    loss_a, plain = grads(None)
    for passes in (1, 2, 4):
        loss_b, ranged = grads(passes)
        assert abs(loss_a - loss_b) <= 1e-4 * abs(loss_a)  # the squared errors are summed with float atomics
        for name in plain:
            # float16 reductions arrive in a different order from run to run
            err = float((plain[name] - ranged[name]).abs().max() / plain[name].abs().max())
            assert err <= 2e-2, f"{name}: {err}"


def test_trainer_refuses_mixed_16_bit_and_float32_parameters():
    enc = HashEncoding(2**10, 4, 3, 2, 4, 32).cuda()
    mlp = FullyFusedMLP(8, 16, 4, depth=1, bias=False).cuda().half()
    with pytest.raises(ValueError):
        NeuralFieldTrainer(enc, mlp)


def test_float32_trainer_goes_through_autograd():
    torch.manual_seed(0)
    enc = HashEncoding(2**10, 4, 3, 2, 4, 32).cuda()
    mlp = FullyFusedMLP(8, 16, 4, depth=2, bias=True).cuda()
    trainer = NeuralFieldTrainer(enc, mlp, lr=1e-2)
    g = torch.Generator().manual_seed(1)
    coords, targets = torch.rand(4096, 3, generator=g).cuda(), torch.rand(4096, 4, generator=g).cuda()
    losses = [float(trainer.step(coords, targets)) for _ in range(10)]
    assert not trainer.direct and losses[-1] < losses[0] and trainer.skipped_elements() == 0


def test_adam_skips_and_counts_non_finite_gradients():
    p = torch.ones(1000, device="cuda", dtype=torch.float16).requires_grad_(True)
    opt = FusedAdam([p], lr=1e-1)
    grad = torch.ones(1000, device="cuda", dtype=torch.float16)
    grad[3], grad[500], grad[999] = float("inf"), float("nan"), -float("inf")
    p.grad = grad
    opt.step()
    assert opt.skipped_elements() == 3
    touched = torch.ones(1000, dtype=torch.bool)
    touched[[3, 500, 999]] = False
    assert torch.isfinite(p).all()
    assert torch.all(p[~touched.cuda()] == 1.0) and torch.all(p[touched.cuda()] < 1.0)
    state = opt.state[p]
    assert torch.isfinite(state["exp_avg"]).all() and torch.isfinite(state["exp_avg_sq"]).all()
    assert float(state["exp_avg"][3]) == 0.0


def test_scale_cast_kernel():
    lib = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(0)
    src = torch.randn(7169, device="cuda", generator=g) * 3.0e4
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        dst = torch.empty(7169, device="cuda", dtype=dtype)
        _lib.check(lib.th_scale_cast(src.data_ptr(), dst.data_ptr(), src.numel(), 2.0**-21, _lib.DTYPE_CODE[dtype], _lib.stream_ptr(src.device)), "th_scale_cast")
        assert torch.equal(dst, (src * 2.0**-21).to(dtype))


def test_cfg3_sized_training_stays_finite_with_headroom():
    # benchmark configuration 3 at full size: 2^21 points, 16 levels x 2 features, T = 2^19, float16,
    # 32 -> 64 -> 64 -> 16.  Thirty steps: the loss stays finite and falls, nothing is skipped, and every
    # stored 16-bit gradient stays below a quarter of float16's range - also when eight ranks' worth is summed.
    torch.manual_seed(0)
    enc = HashEncoding(2**19, 16, 3, 2, 16, 2048)
    with torch.no_grad():
        enc.embeddings.uniform_(-1e-4, 1e-4)
    mlp = FullyFusedMLP(32, 64, 16, depth=2, bias=False)
    trainer = NeuralFieldTrainer(enc.cuda().half(), mlp.cuda().half(), lr=1e-2, betas=(0.9, 0.99), eps=1e-15)
    g = torch.Generator(device="cuda").manual_seed(1234)
    n = 2**21
    coords = torch.rand(n, 3, device="cuda", generator=g)
    targets = torch.rand(n, 16, device="cuda", generator=g).half()
    limit = 0.25 * torch.finfo(torch.float16).max
    losses, worst_mlp = [], 0.0
    for _ in range(30):
        losses.append(float(trainer.step(coords, targets)))
        st = trainer._state
        worst_mlp = max(worst_mlp, float(st.mlp_grad.float().abs().max()))  # the MLP part is overwritten, not cleared
        assert torch.isfinite(st.table_m).all() and torch.isfinite(st.mlp_m).all()
    assert all(map(lambda v: v == v and v < 1.0, losses)), losses
    assert losses[-1] < 0.5 * losses[0], losses
    assert trainer.skipped_elements() == 0
    # Adam clears the table part as it consumes it: look at the table gradient of one more backward at the
    # final parameters, through the layers' autograd functions with the same loss scale
    scale = trainer.grad_out_scale
    feats = enc(coords)
    pred = mlp(feats.unsqueeze(0)).squeeze(0)
    grad_out, _ = mse_grad(pred, targets, scale)
    pred.backward(grad_out)
    worst_table = float(enc.embeddings.grad.float().abs().max())
    assert 8 * worst_table < limit, worst_table     # eight ranks summing their table gradients
    assert 8 * worst_mlp < limit, worst_mlp          # eight ranks summing their (mean) MLP gradients
    assert scale == 1.0 / 8


# ---- measurement entry points ---------------------------------------------------------------------


def test_launch_counter():
    lib = _lib.lib()
    src = torch.ones(100, device="cuda")
    dst = torch.empty(100, device="cuda")
    before = lib.th_launch_count()
    for _ in range(3):
        _lib.check(lib.th_scale_cast(src.data_ptr(), dst.data_ptr(), 100, 1.0, 0, _lib.stream_ptr(src.device)), "th_scale_cast")
    assert lib.th_launch_count() - before == 3
    # argument errors are reported, not launched
    assert lib.th_scale_cast(src.data_ptr(), dst.data_ptr(), 100, 1.0, 9, _lib.stream_ptr(src.device)) < 0
    assert lib.th_launch_count() - before == 3


def test_no_stream_synchronisation_in_the_encoding_calls():
    # Forward and backward only enqueue work: the hash primes are read from the device once per
    # tensor, not on every call (a read would serialise the host behind the GPU).
    from triton_helpers_b200.layers.hash_encoding import HashEncoding

    enc = HashEncoding(2**14, 8, 3, 2, 16, 256).cuda()
    x = torch.rand(4096, 3, device="cuda")
    enc(x).sum().backward()  # first call may read `pi`
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        out = enc(x)
        out.backward(torch.ones_like(out))
    finally:
        torch.cuda.set_sync_debug_mode("default")
