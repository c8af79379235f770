r"""Host logic of the data-parallel step on CPU ranks (gloo, world_size 2): sharding, bucketing,
the gradient all-reduce wrapper, and the identity "sum of per-shard gradients = full-batch gradient"
using the CPU port of the training step."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from triton_helpers_b200.parallel import (
    PendingReduce,
    allreduce_gradients,
    gradient_scales,
    init_from_env,
    level_passes,
    plan_buckets,
    shard_bounds,
)


def test_shard_bounds_cover_everything_once():
    for n, world in [(10, 3), (2**21, 8), (7, 8), (0, 2)]:
        spans = [shard_bounds(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1


def test_plan_buckets():
    assert plan_buckets([10, 20, 30], 100) == [[0, 1, 2]]
    assert plan_buckets([10, 2000, 30], 100) == [[1], [0, 2]]
    assert plan_buckets([60, 60, 60], 100) == [[0], [1], [2]]
    assert plan_buckets([], 100) == []


def test_level_passes_cover_every_level_once_finest_first():
    from triton_helpers_b200.layers.hash_encoding.helpers import level_geometry

    for rows in (level_geometry(16, 2**19, 3, 16, 2048).rows, level_geometry(16, 2**22, 3, 16, 4096).rows, [7] * 8, [3, 3]):
        for n in (1, 2, 3, 4, 9):
            passes = level_passes(rows, n)
            assert 1 <= len(passes) <= n
            assert passes[0][1] == len(rows) and passes[-1][0] == 0
            assert all(a[0] == b[1] for a, b in zip(passes, passes[1:]))  # consecutive, descending
            assert all(b % 4 == 0 for b, _ in passes)
    assert level_passes(level_geometry(16, 2**19, 3, 16, 2048).rows, 2) == [(8, 16), (0, 8)]


def test_pending_reduce_is_a_noop_without_a_process_group():
    g = torch.ones(4)
    pending = PendingReduce()
    pending.start([g, None])
    pending.finish()
    assert torch.equal(g, torch.ones(4))


def test_allreduce_is_a_noop_without_a_process_group():
    g = torch.ones(4)
    allreduce_gradients([g, None])
    assert torch.equal(g, torch.ones(4))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    got_rank, got_world, _ = init_from_env("gloo")
    assert (got_rank, got_world) == (rank, world)
    try:
        # 1. buckets: one large tensor reduced in place, small ones packed, a second dtype, a strided view
        big = torch.full((1 << 16,), float(rank + 1))
        small = [torch.full((7,), float(rank)), torch.full((3, 5), 2.0 * rank)]
        other = torch.full((9,), rank + 1, dtype=torch.float64)
        strided = torch.full((8, 8), float(rank + 1))[:, ::2]
        allreduce_gradients([big, *small, None, other, strided], bucket_bytes=1 << 12)
        total = sum(range(1, world + 1))
        assert torch.all(big == total) and torch.all(other == total) and torch.all(strided == total)
        assert torch.all(small[0] == sum(range(world))) and torch.all(small[1] == 2.0 * sum(range(world)))

        # 1b. the same sums started asynchronously, range by range, and awaited once
        table = torch.full((1000, 2), float(rank + 1))
        tiny = [torch.full((5,), float(rank)), torch.full((2, 3), 3.0 * rank)]
        pending = PendingReduce(bucket_bytes=1 << 12)
        pending.start(tiny)
        pending.start([table[600:]])
        pending.start([table[:600]])
        pending.finish()
        assert torch.all(table == total)
        assert torch.all(tiny[0] == sum(range(world))) and torch.all(tiny[1] == 3.0 * sum(range(world)))

        # 2. data parallel identity with the CPU port of the training step: mean-loss gradients of the
        #    two half batches, summed and halved, equal the full-batch gradient
        from oracle.training_step import CpuNeuralField, make_batch

        kw = dict(levels=4, table_cap=2**10, n_min=4, n_max=64, d_hidden=16, d_out=4, depth=2, seed=0)
        coords, targets = make_batch(512, d_out=4, seed=1)
        begin, end = shard_bounds(512, rank, world)
        local = CpuNeuralField(**kw)
        loss = torch.nn.functional.mse_loss(local.predict(coords[begin:end]), targets[begin:end])
        loss.backward()
        grads = [p.grad for p in local.params.values()]
        allreduce_gradients(grads)
        full = CpuNeuralField(**kw)
        torch.nn.functional.mse_loss(full.predict(coords), targets).backward()
        for g, p in zip(grads, full.params.values()):
            torch.testing.assert_close(g / world, p.grad, rtol=1e-4, atol=1e-7)
        results[rank] = True
    finally:
        dist.destroy_process_group()


def test_gradient_scales_recover_the_mean_loss_gradient():
    # one rank, float64: the three factors undo the loss scale and the normalisation exactly
    g = torch.Generator().manual_seed(0)
    rows, d_out, s = 1000, 4, 1.0 / 8
    pred, target = torch.randn(rows, d_out, generator=g, dtype=torch.float64), torch.rand(rows, d_out, generator=g, dtype=torch.float64)
    w = torch.randn(d_out, 3, generator=g, dtype=torch.float64, requires_grad=True)
    feats = torch.randn(rows, 3, generator=g, dtype=torch.float64)
    ((feats @ w.T + pred - target) ** 2).mean().backward()
    stored_sum = ((feats @ w.T + pred - target).detach() * s).T @ feats  # what a backward fed (diff * s) accumulates
    cast, table_scale, mlp_scale = gradient_scales(rows, 1, d_out, s)
    torch.testing.assert_close(stored_sum * cast * mlp_scale, w.grad)
    torch.testing.assert_close(stored_sum * table_scale, w.grad)
    # more ranks: every factor that multiplies a SUM over ranks carries 1 / world
    assert gradient_scales(rows, 4, d_out, s)[2] == mlp_scale / 4 and gradient_scales(rows, 4, d_out, s)[0] == cast


def _sum_worker(rank: int, world: int, port: int, results):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    init_from_env("gloo")
    try:
        # Per-rank float32 sums of the size the cfg 3 step produces (|dW| ~ 2e4 with 2^21 rows and loss scale
        # 1/16).  Rounded to float16 as they are, four of them overflow; normalised first they do not.
        rows, s, d_out = 2**21, 1.0 / 16, 16
        g = torch.Generator().manual_seed(7)
        shape = torch.rand(64, 64, generator=g) + 0.5            # same on every rank
        sums = shape * 2.0e4 * (1.0 + 0.1 * rank)                # this rank's float32 workspace
        cast, _, mlp_scale = gradient_scales(rows, world, d_out, s)
        table = torch.full((1001, 2), float(rank + 1), dtype=torch.float16)
        flat = torch.zeros(2016 + 64 * 64, dtype=torch.float16)  # [table | pad | MLP], as the trainer lays it out
        flat[:2002] = table.reshape(-1)
        flat[2016:] = (sums * cast).to(torch.float16).reshape(-1)  # what th_scale_cast writes
        pending = PendingReduce(bucket_bytes=0)
        pending.start([flat])
        pending.finish()
        got = flat[2016:].float().view(64, 64) * mlp_scale
        want = sum(shape.double() * 2.0e4 * (1.0 + 0.1 * r) for r in range(world)) * 2.0 / (rows * world * d_out * s)
        assert torch.isfinite(flat).all()
        torch.testing.assert_close(got.double(), want, rtol=4e-3, atol=0)
        assert torch.all(flat[:2002] == sum(range(1, world + 1)))
        # the convention this replaces: unnormalised float16 sums
        naive = sums.to(torch.float16)
        dist.all_reduce(naive)
        assert not torch.isfinite(naive).all()
        results[rank] = True
    finally:
        dist.destroy_process_group()


def test_four_rank_gloo_sum_of_large_gradients_in_float16():
    world = 4
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_sum_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {r: True for r in range(world)}


def test_two_rank_gloo_gradient_sum():
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {0: True, 1: True}
