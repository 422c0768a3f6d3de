"""Host-side partitioning of the path across GPUs (one process per GPU).

Two natural splits exist and nothing else is invented:
  * independent decode sequences -> ranks, no collective (``shard_sequences``);
  * KV-head groups -> ranks for prefill / batched decode of one sequence set: rank r owns KV heads
    [r*Hkv/N, (r+1)*Hkv/N) and the query heads that map onto them; each rank writes its output
    head-major, so ONE all-gather in rank order yields the final [n_head][n_tok][head_dim] tensor
    (``HeadShardedPrefill`` / ``FusedHeadShardedPrefill`` for prefill, ``HeadShardedDecode`` /
    ``FusedHeadShardedDecode`` for a batched decode step).
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


class HeadShardedPrefill:
    """Head-sharded causal prefill of one sequence with the all-gather of head outputs overlapped.

    The query range is cut into ``n_chunks`` row chunks.  Chunks are computed from the LAST (most
    keys, most work) to the FIRST (cheapest); as soon as a chunk's local heads are done its
    all-gather starts on a side stream while the next chunk computes, so only the gather of the
    cheapest chunk is exposed.  Result layout: ``[n_chunks][n_head][chunk_rows][head_dim]`` fp16
    -- per chunk, rank-order concatenation of the head-major local outputs is the final layout.
    K/V of the whole sequence must have been appended to this rank's KV pool slice before.
    """

    def __init__(self, ctx, kv, shape, n_tok: int, n_chunks: int, device, world: int | None = None):
        if n_tok % n_chunks != 0:
            raise ValueError("n_tok must divide into n_chunks")
        self.ctx, self.kv, self.shape = ctx, kv, shape
        self.n_tok, self.n_chunks, self.rows = n_tok, n_chunks, n_tok // n_chunks
        self.world = world if world is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        hd = shape.head_dim
        self.local = torch.empty((n_chunks, shape.n_head, self.rows, hd), dtype=torch.float16, device=device)
        self.full = torch.empty((n_chunks, shape.n_head * self.world, self.rows, hd), dtype=torch.float16,
                                device=device)
        self.comm_stream = torch.cuda.Stream(device=device)
        self.events = [torch.cuda.Event() for _ in range(n_chunks)]

    def run(self, q: torch.Tensor, block_table: torch.Tensor, layer: int = 0) -> torch.Tensor:
        """q: [n_tok, n_head_local, hd] (this rank's query heads).  Returns the gathered tensor; the
        caller's stream is made to wait for the last gather."""
        main = torch.cuda.current_stream()
        self.comm_stream.wait_stream(main)  # earlier readers of `full` on the main stream are done
        for c in range(self.n_chunks - 1, -1, -1):
            lo = c * self.rows
            self.ctx.attn_prefill(self.kv, layer, self.shape, q[lo:lo + self.rows], lo, block_table,
                                  self.local[c].permute(1, 0, 2))
            if self.world > 1:
                self.events[c].record(main)
                with torch.cuda.stream(self.comm_stream):
                    self.comm_stream.wait_event(self.events[c])
                    dist.all_gather_into_tensor(self.full[c], self.local[c])
            else:
                self.full[c].copy_(self.local[c])
        main.wait_stream(self.comm_stream)
        return self.full


class FusedHeadShardedPrefill:
    """Head-sharded causal prefill with the all-gather of head outputs fused INTO the attention kernel.

    Every rank allocates the full ``[n_head][n_tok][head_dim]`` fp16 result in symmetric memory (the same
    buffer on every GPU, each mapped into the others' address spaces).  A rank's prefill kernel stores
    each finished output tile of its own heads into its slice of the buffer on ALL ranks -- plain
    stores to peer memory over NVLink, spread over the whole run of the kernel -- so when the kernels
    end the gather is already done; only a barrier remains.  No collective kernel is launched.
    """

    def __init__(self, ctx, kv, shape, n_tok: int, n_head_total: int, device, group=None):
        import torch.distributed._symmetric_memory as symm

        self.ctx, self.kv, self.shape, self.n_tok = ctx, kv, shape, n_tok
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        hd = shape.head_dim
        if self.world > 1:
            self.full = symm.empty((n_head_total, n_tok, hd), dtype=torch.float16, device=device)
            self.hdl = symm.rendezvous(self.full, group if group is not None else dist.group.WORLD)
            ptrs = list(self.hdl.buffer_ptrs)
        else:
            self.full = torch.empty((n_head_total, n_tok, hd), dtype=torch.float16, device=device)
            self.hdl, ptrs = None, [self.full.data_ptr()]
        q_lo = self.rank * shape.n_head
        self.local = self.full[q_lo:q_lo + shape.n_head]           # [n_head_local, n_tok, hd]
        byte_off = q_lo * n_tok * hd * 2
        self.peer_ptrs = [ptrs[p] + byte_off for p in range(self.world) if p != self.rank]

    def run(self, q: torch.Tensor, block_table: torch.Tensor, layer: int = 0) -> torch.Tensor:
        self.ctx.attn_prefill_bcast(self.kv, layer, self.shape, q, 0, block_table, self.local.permute(1, 0, 2),
                                    self.peer_ptrs)
        if self.hdl is not None:
            self.hdl.barrier()  # every rank's kernel has finished: all slices of `full` are in place
        return self.full


class HeadShardedDecode:
    """One batched decode step with KV heads split across ranks and ONE all-gather of the head outputs.

    Rank r holds KV heads [r*Hkv/N, (r+1)*Hkv/N) of EVERY sequence's pages (same block tables on all ranks, a pool
    with Hkv/N heads) and runs the split-KV decode on the n_head/N query heads that map onto them -- N copies of the
    reference's single-GPU gpuAttentionDecode (src/hippo_leap/backends/naive.nim:4714-4717), each over 1/N of the cache
    bytes.  Output is head-major ``[n_head/N][batch][head_dim]``, so the rank-order concatenation of one
    ``all_gather_into_tensor`` is the final ``[n_head][batch][head_dim]``.  ``shape`` is the LOCAL shape.
    """

    def __init__(self, ctx, kv, shape, batch: int, device, world: int | None = None, dtype=torch.float32):
        self.ctx, self.kv, self.shape, self.batch = ctx, kv, shape, batch
        self.world = world if world is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        self.local = torch.empty((shape.n_head, batch, shape.head_dim), dtype=dtype, device=device)
        self.full = torch.empty((shape.n_head * self.world, batch, shape.head_dim), dtype=dtype, device=device)

    def run(self, q, k_new, v_new, ctx_lens, max_ctx: int, block_tables, layer: int = 0) -> torch.Tensor:
        """q [batch, n_head_local, hd], k_new / v_new [batch, n_head_kv_local, hd]: this rank's heads of the new token
        of every sequence (in a full model they come from column-sharded projections).  Appends, attends, gathers."""
        self.ctx.kv_append_batch(self.kv, layer, self.shape, k_new, v_new, ctx_lens, block_tables)
        self.ctx.attn_decode(self.kv, layer, self.shape, q, ctx_lens, max_ctx, block_tables, self.local.permute(1, 0, 2))
        if self.world > 1:
            dist.all_gather_into_tensor(self.full, self.local)
        else:
            self.full.copy_(self.local)
        return self.full


class FusedHeadShardedDecode:
    """The same step with the gather fused into the decode kernels: the full ``[n_head][batch][head_dim]`` result
    lives in symmetric memory and every rank's decode / combine kernel stores its finished rows into its head slice
    on ALL ranks (plain stores to peer memory over NVLink).  No collective kernel runs; a barrier remains."""

    def __init__(self, ctx, kv, shape, batch: int, n_head_total: int, device, group=None, dtype=torch.float32):
        import torch.distributed._symmetric_memory as symm

        self.ctx, self.kv, self.shape, self.batch = ctx, kv, shape, batch
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        hd = shape.head_dim
        if self.world > 1:
            self.full = symm.empty((n_head_total, batch, hd), dtype=dtype, device=device)
            self.hdl = symm.rendezvous(self.full, group if group is not None else dist.group.WORLD)
            ptrs = list(self.hdl.buffer_ptrs)
        else:
            self.full = torch.empty((n_head_total, batch, hd), dtype=dtype, device=device)
            self.hdl, ptrs = None, [self.full.data_ptr()]
        q_lo = self.rank * shape.n_head
        self.local = self.full[q_lo:q_lo + shape.n_head]
        byte_off = q_lo * batch * hd * self.full.element_size()
        self.peer_ptrs = [ptrs[p] + byte_off for p in range(self.world) if p != self.rank]

    def run(self, q, k_new, v_new, ctx_lens, max_ctx: int, block_tables, layer: int = 0) -> torch.Tensor:
        self.ctx.kv_append_batch(self.kv, layer, self.shape, k_new, v_new, ctx_lens, block_tables)
        self.ctx.attn_decode_bcast(self.kv, layer, self.shape, q, ctx_lens, max_ctx, block_tables,
                                   self.local.permute(1, 0, 2), self.peer_ptrs)
        if self.hdl is not None:
            self.hdl.barrier()  # every rank's kernels have finished: all slices of `full` are in place
        return self.full
