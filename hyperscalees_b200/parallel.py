"""Population sharding across the GPUs of one node.

The population step shards by contiguous, pair-aligned member ranges: rank g
owns thread ids [lo_g, hi_g) with lo_g even, so the two members of an
antithetic pair always sit on the same GPU.  Every rank regenerates its own
members' noise from (key, epoch, thread id) — the same rule as the reference's
multi-GPU script (llm_experiments/snn_mnist_train_multi_gpu.py:146-149,
186-205) — so the only exchange of a step is the all-gather of the raw fitness
vector; afterwards every rank holds the full vector, normalises it identically
and applies the same update.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n_pop: int, rank: int, world: int) -> Tuple[int, int]:
    """Members [lo, hi) owned by `rank`: whole antithetic pairs, sizes differing by at most one pair."""
    if n_pop % 2 != 0:
        raise ValueError("the population must consist of whole antithetic pairs (n_pop even)")
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    pairs = n_pop // 2
    base, extra = divmod(pairs, world)
    lo_pair = rank * base + min(rank, extra)
    hi_pair = lo_pair + base + (1 if rank < extra else 0)
    return 2 * lo_pair, 2 * hi_pair


def shard_sizes(n_pop: int, world: int) -> List[int]:
    return [hi - lo for lo, hi in (shard_range(n_pop, r, world) for r in range(world))]


def allgather_fitness(local: torch.Tensor, n_pop: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather the per-member raw fitness of every shard into the full (n_pop,) vector, in
    thread-id order.  Works with NCCL (CUDA tensors) and gloo (CPU tensors)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        if local.numel() != n_pop:
            raise ValueError("single-rank fitness vector must cover the whole population")
        return local
    rank = dist.get_rank(group)
    sizes = shard_sizes(n_pop, world)
    if local.numel() != sizes[rank]:
        raise ValueError(f"rank {rank} owns {sizes[rank]} members but passed {local.numel()} fitness values")
    if len(set(sizes)) == 1:
        out = torch.empty(n_pop, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    # shards of unequal size: pad every shard to the largest one, gather, drop the padding
    m = max(sizes)
    padded = torch.zeros(m, dtype=local.dtype, device=local.device)
    padded[:local.numel()] = local
    out = torch.empty(world * m, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    return torch.cat([out[r * m:r * m + sizes[r]] for r in range(world)])


def allreduce_grads(grads: List[torch.Tensor], group: Optional[dist.ProcessGroup] = None) -> None:
    """Optional second exchange: sum partial gradients computed per shard (each rank called
    the update with its own first_thread and n_total = n_pop).  The sum order is NCCL's; ranks
    that need bit-identical parameters should use the replicated update instead."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        for g in grads:
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
