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
