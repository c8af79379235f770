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
    assert all(p.grad is None for p in trainer.parameters())
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


def test_backward_in_level_passes_matches_the_autograd_path():
    # the backward a multi-rank run may take (encoding backward range by range, sums started in
    # between), here on one rank where the sums are no-ops: same gradients as the single-pass backward
    torch.manual_seed(3)
    enc = HashEncoding(2**12, 8, 3, 2, 8, 128)
    mlp = FullyFusedMLP(16, 32, 4, depth=2, bias=False)
    trainer = NeuralFieldTrainer(enc.cuda().half(), mlp.cuda().half(), lr=1e-2)
    g = torch.Generator().manual_seed(4)
    coords = torch.rand(8192, 3, generator=g).cuda()
    targets = torch.rand(8192, 4, generator=g).cuda().half()

    def grads(run):
        for p in trainer.parameters():
            p.grad = None
        _, loss_sum = run()
        return float(loss_sum), {n: p.grad.float().clone() for n, p in trainer.named_parameters()}

    loss_a, plain = grads(lambda: trainer._backward_through_autograd(coords, targets))
    for passes in (1, 2, 4):
        loss_b, ranged = grads(lambda: trainer._backward_in_level_passes(coords, targets, passes))
        assert abs(loss_a - loss_b) <= 1e-4 * abs(loss_a)  # the squared errors are summed with float atomics
        for name in plain:
            # float16 reductions arrive in a different order from run to run
            err = float((plain[name] - ranged[name]).abs().max() / plain[name].abs().max())
            assert err <= 2e-2, f"{name}: {err}"


# ---- measurement entry points ---------------------------------------------------------------------


def test_launch_counter_and_l2_probe():
    import ctypes

    lib = _lib.lib()
    device = torch.device("cuda", 0)
    buf = torch.zeros(8 * 2**20, dtype=torch.uint8, device=device)
    sink = torch.zeros(1, dtype=torch.int32, device=device)
    before = lib.th_launch_count()
    for mode, expect in ((0, 8 * 2**20 * 3), (1, None), (2, None)):
        work = ctypes.c_int64(0)
        _lib.check(lib.th_probe_l2(buf.data_ptr(), buf.numel(), mode, 3, sink.data_ptr(), ctypes.byref(work), _lib.stream_ptr(device)), "th_probe_l2")
        assert work.value > 0 and (expect is None or work.value == expect)
    torch.cuda.synchronize()
    assert lib.th_launch_count() - before == 3
    # argument errors are reported, not launched
    assert lib.th_probe_l2(buf.data_ptr(), buf.numel(), 7, 1, sink.data_ptr(), None, _lib.stream_ptr(device)) < 0
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
