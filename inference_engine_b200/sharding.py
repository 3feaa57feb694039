"""Sequence sharding of the attention path across the GPUs of one box.

Every sequence's quantize-on-write and attention touch only that sequence's pages, so the path
shards by sequence with no collective on the data path: one process per GPU, each with its own
page pool and block tables.  Sequences are assigned so that the bytes of KV cache each GPU has to
stream per step are balanced (longest-processing-time-first: sort by context, give each to the
least-loaded GPU).  The only collective is a verification-time all_gather of outputs.

The reference engine is single-GPU (engine.py:51); this is the multi-GPU layer added around the
same per-sequence operators."""
from __future__ import annotations

import heapq
from dataclasses import dataclass

import torch
import torch.distributed as dist

KV_BYTES_PER_TOKEN_PER_LAYER = 8 * (2 * 128 + 8)  # 8 KV heads x (128 K codes + 128 V codes + 2 fp32 scales)


@dataclass
class ShardPlan:
    world_size: int
    owner: list[int]  # owner[i] = rank that holds sequence i
    local: list[list[int]]  # local[r] = global sequence ids of rank r, in local order
    load: list[int]  # load[r] = KV tokens rank r streams per step

    def imbalance(self) -> float:
        """max load / mean load (1.0 = perfectly balanced)."""
        mean = sum(self.load) / max(1, self.world_size)
        return max(self.load) / mean if mean > 0 else 1.0


def plan_shards(context_lens, world_size: int) -> ShardPlan:
    """Longest-processing-time-first assignment of sequences to ranks by KV tokens.  Deterministic
    (ties broken by sequence id, then by rank), so every rank computes the same plan locally."""
    order = sorted(range(len(context_lens)), key=lambda i: (-int(context_lens[i]), i))
    heap = [(0, r) for r in range(world_size)]
    owner = [0] * len(context_lens)
    local: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        load, r = heapq.heappop(heap)
        owner[i] = r
        local[r].append(i)
        heapq.heappush(heap, (load + int(context_lens[i]), r))
    load = [sum(int(context_lens[i]) for i in ids) for ids in local]
    return ShardPlan(world_size, owner, local, load)


def gather_outputs(local_out: torch.Tensor, plan: ShardPlan, rank: int, group=None) -> torch.Tensor:
    """all_gather the per-rank outputs [len(plan.local[rank]), ...] and put them back in global
    sequence order.  Verification only: never on the timed path."""
    world = plan.world_size
    width = max(len(ids) for ids in plan.local)
    pad = torch.zeros((width,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    pad[: local_out.shape[0]] = local_out
    if world > 1:
        parts = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(parts, pad, group=group)
    else:
        parts = [pad]
    out = torch.zeros((len(plan.owner),) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    for r, ids in enumerate(plan.local):
        if ids:
            out[torch.as_tensor(ids, device=out.device)] = parts[r][: len(ids)]
    return out
