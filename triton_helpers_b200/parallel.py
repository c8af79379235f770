r"""Data parallelism over points: one process per GPU, replicated parameters, summed gradients.

The fused operators are embarrassingly parallel over points; the only exchange in a training
step is the sum of the parameter gradients (hash table + MLP weights), done once per step with
``torch.distributed.all_reduce`` (NCCL over NVLink on GPUs, gloo in the CPU tests).  Kernels
never read peer memory.  triton_helpers has no distributed code; this is the whole of it here.
"""
import os
from typing import Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def init_from_env(backend: Optional[str] = None) -> Tuple[int, int, int]:
    r"""Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun's
    environment).  Returns ``(rank, world_size, local_rank)``; a single process needs no group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
            dist.init_process_group(backend, device_id=torch.device("cuda", local_rank))
        else:
            dist.init_process_group(backend)
    return rank, world, local_rank


def shard_bounds(n_items: int, rank: int, world_size: int) -> Tuple[int, int]:
    r"""Contiguous, near-equal slice ``[begin, end)`` of ``n_items`` owned by ``rank``."""
    base, extra = divmod(n_items, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def plan_buckets(sizes_bytes: Sequence[int], bucket_bytes: int) -> List[List[int]]:
    r"""Greedy grouping of tensor indices into buckets of at most ``bucket_bytes`` (a tensor larger
    than that gets a bucket of its own).  Small tensors share one flat all-reduce; large ones are
    reduced in place."""
    buckets: List[List[int]] = []
    current, current_bytes = [], 0
    for i, size in enumerate(sizes_bytes):
        if size >= bucket_bytes:
            buckets.append([i])
            continue
        if current and current_bytes + size > bucket_bytes:
            buckets.append(current)
            current, current_bytes = [], 0
        current.append(i)
        current_bytes += size
    if current:
        buckets.append(current)
    return buckets


def allreduce_gradients(
    grads: Iterable[Tensor], group: Optional[dist.ProcessGroup] = None, bucket_bytes: int = 1 << 20
) -> None:
    r"""Sum ``grads`` over all ranks, in place.

    Tensors of at least ``bucket_bytes`` (the hash-table gradient) are reduced directly; smaller
    ones of the same dtype (the MLP gradients, a few KB each) are packed into one flat buffer so
    they cost one collective instead of one each.  No-op without an initialised process group.
    """
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    grads = [g for g in grads if g is not None]
    by_dtype = {}
    for g in grads:
        by_dtype.setdefault(g.dtype, []).append(g)
    for same in by_dtype.values():
        sizes = [g.numel() * g.element_size() for g in same]
        for bucket in plan_buckets(sizes, bucket_bytes):
            if len(bucket) == 1:
                g = same[bucket[0]]
                if g.is_contiguous():
                    dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
                else:
                    flat = g.contiguous()
                    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
                    g.copy_(flat)
                continue
            members = [same[i] for i in bucket]
            flat = torch.cat([m.reshape(-1) for m in members])
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
            offset = 0
            for m in members:
                m.copy_(flat[offset : offset + m.numel()].view_as(m))
                offset += m.numel()


def gradient_scales(rows: int, world_size: int, d_out: int, grad_out_scale: float) -> Tuple[float, float, float]:
    r"""The three factors that tie the flat 16-bit gradient buffer of a data-parallel step to the true
    gradient of ``mean((pred - target)^2)`` over the global batch of ``rows * world_size`` points with
    ``d_out`` values each, when the backward pass was fed ``(pred - target) * grad_out_scale``:

    * ``cast_scale``: multiplies the float32 sums over the local rows that the MLP backward leaves in its
      workspace before they are rounded to 16 bits - ``1 / (rows * grad_out_scale)``, i.e. the buffer holds
      the mean of the unscaled gradient.  Sums over 2^21 rows reach 1e4..1e5 and would overflow float16
      once four ranks are added up; means of any number of rows stay of order one.
    * ``table_adam_scale``: multiplies the summed table gradient (which holds ``grad_out_scale * sum``).
    * ``mlp_adam_scale``: multiplies the summed MLP gradient (a sum of per-rank means).
    """
    per_value = 2.0 / (world_size * d_out)
    return 1.0 / (rows * grad_out_scale), per_value / (rows * grad_out_scale), per_value


def level_passes(level_rows: Sequence[int], n_passes: int, align: int = 4) -> List[Tuple[int, int]]:
    r"""Cuts levels ``0 .. len(level_rows)`` into at most ``n_passes`` consecutive ranges holding about
    equal numbers of table rows, with boundaries at multiples of ``align`` levels (the backward kernel
    handles four levels per register group), listed FINEST FIRST: the fine levels hold most rows, so
    their all-reduce is the one worth starting early."""
    levels = len(level_rows)
    if n_passes <= 1 or levels <= align:
        return [(0, levels)]
    total = sum(level_rows)
    cuts, acc, target = [], 0, total / n_passes
    for l in range(levels - 1, 0, -1):  # walk down from the finest level
        acc += level_rows[l]
        if l % align == 0 and acc >= target * (len(cuts) + 1) and len(cuts) < n_passes - 1:
            cuts.append(l)
    bounds = [levels] + cuts + [0]
    return [(bounds[i + 1], bounds[i]) for i in range(len(bounds) - 1)]


class PendingReduce:
    r"""Sums of gradient tensors over all ranks that have been started and not yet awaited.

    ``start`` queues an asynchronous all-reduce of each tensor (small tensors of one dtype share a flat
    buffer, as in ``allreduce_gradients``) behind the work already queued on the current stream;
    ``finish`` makes the current stream wait for all of them and copies flat buffers back.  Between
    the two the caller keeps launching kernels that do not touch those tensors."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, bucket_bytes: int = 1 << 20):
        self.group, self.bucket_bytes = group, bucket_bytes
        self.active = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self._works = []
        self._unpack = []

    def start(self, grads: Iterable[Tensor]) -> None:
        if not self.active:
            return
        grads = [g for g in grads if g is not None]
        by_dtype = {}
        for g in grads:
            by_dtype.setdefault(g.dtype, []).append(g)
        for same in by_dtype.values():
            sizes = [g.numel() * g.element_size() for g in same]
            for bucket in plan_buckets(sizes, self.bucket_bytes):
                members = [same[i] for i in bucket]
                if len(members) == 1 and members[0].is_contiguous():
                    self._works.append(dist.all_reduce(members[0], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
                    continue
                flat = torch.cat([m.reshape(-1) for m in members])
                self._works.append(dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
                self._unpack.append((flat, members))

    def finish(self) -> None:
        for work in self._works:
            work.wait()
        for flat, members in self._unpack:
            offset = 0
            for m in members:
                m.copy_(flat[offset : offset + m.numel()].view_as(m))
                offset += m.numel()
        self._works, self._unpack = [], []
