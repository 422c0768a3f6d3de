"""Host-side partitioning of the path across GPUs (one process per GPU).

Two natural splits exist and nothing else is invented:
  * independent decode sequences -> ranks, no collective (``shard_sequences``);
  * KV-head groups -> ranks for prefill / batched decode of one sequence set: rank r owns KV heads
    [r*Hkv/N, (r+1)*Hkv/N) and the query heads that map onto them; each rank writes its output
    head-major, so ONE all-gather in rank order yields the final [n_head][n_tok][head_dim] tensor.
The reference has no multi-GPU code at all (one stream, one global lock:
src/hippo_leap/backends/naive.nim:237-243, src/hippo_leap/inference.nim:53-54).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from .synth import shard_longest_first


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    kv_lo: int
    kv_hi: int
    q_lo: int
    q_hi: int

    @property
    def n_head_kv(self) -> int:
        return self.kv_hi - self.kv_lo

    @property
    def n_head(self) -> int:
        return self.q_hi - self.q_lo


def head_shard(rank: int, world: int, n_head: int, n_head_kv: int) -> HeadShard:
    """KV heads and query heads owned by ``rank``; raises ValueError when they do not divide."""
    if n_head % n_head_kv != 0:
        raise ValueError("GQA requires head_count divisible by head_count_kv")
    if n_head_kv % world != 0:
        raise ValueError(f"{n_head_kv} KV heads do not divide over {world} ranks")
    per = n_head_kv // world
    group = n_head // n_head_kv
    return HeadShard(rank, world, rank * per, (rank + 1) * per, rank * per * group, (rank + 1) * per * group)


def shard_sequences(ctx_lens, world: int):
    """Greedy longest-first assignment of sequence indices to ranks (balances KV bytes)."""
    return shard_longest_first(np.asarray(ctx_lens), world)


def gather_heads(out_local: torch.Tensor, full: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather of head-major outputs: out_local [n_head/N, n_tok, hd] -> [n_head, n_tok, hd]."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    if full is None:
        full = torch.empty((out_local.shape[0] * world,) + tuple(out_local.shape[1:]), dtype=out_local.dtype,
                           device=out_local.device)
    if world == 1:
        full.copy_(out_local)
        return full
    dist.all_gather_into_tensor(full, out_local.contiguous())
    return full


def max_over_ranks(value: float, device) -> float:
    """Timing rule for every multi-GPU number: the slowest rank decides."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
