"""Multi-GPU plumbing: one process per GPU, structures sharded across ranks, no collective on the hot path.

Structures never interact (edges never cross structures, src/mlcg/neighbor_list/neighbor_list.py:89-91), so
energy / force evaluation and simulation replicas shard by contiguous blocks of structures.  The only
collective is the gradient all-reduce of data-parallel force-matching training (what Lightning's DDP strategy
does for mlcg, examples/input_yamls/slurm_example/train.yaml:9): one flat bucket, sum then divide.
"""
from typing import Iterable, Tuple

import torch
import torch.distributed as dist


def shard_range(num_structures: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous block of structures owned by ``rank`` (sizes differ by at most one)."""
    base, rem = divmod(num_structures, world_size)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group=None) -> None:
    """Average ``.grad`` over ranks through one flat buffer (the whole SchNet is ~1 MB of gradients)."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    flat /= dist.get_world_size(group)
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()


def max_over_ranks(value: float, device, group=None) -> float:
    """Slowest rank's time: what a multi-GPU throughput number has to be computed from."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t[0])
