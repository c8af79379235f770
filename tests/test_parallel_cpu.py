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
