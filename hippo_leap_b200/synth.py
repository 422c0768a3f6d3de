"""Seeded synthetic workloads with the shapes of the five benchmark configurations.

No model file or dataset is involved: activations are N(0,1) draws from
``numpy.random.Generator(PCG64(seed))`` so that the CUDA path, the CPU oracle and the CPU
baseline all read identical bytes.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .runtime import theta_llama3_scale, theta_table


@dataclass(frozen=True)
class AttnConfig:
    name: str
    n_head: int
    n_head_kv: int
    head_dim: int
    rope_base: float
    layers: int = 1
    prefill: int = 0          # prompt tokens
    decode_steps: int = 0
    llama3_scaling: bool = False
    qk_norm: bool = False
    rms_eps: float = 1e-6
    bf16_range: bool = False  # activations rounded to bf16 before use
    fp16_inputs: bool = False  # Q / K / V handed to the kernels as fp16 (config 5), float32 otherwise
    batch: int = 1            # concurrent sequences (batched decode)
    ctx_range: tuple = (0, 0)
    block_tokens: int = 16
    seed: int = 0

    @property
    def group(self) -> int:
        return self.n_head // self.n_head_kv

    def theta(self) -> np.ndarray:
        th = theta_table(self.head_dim, self.rope_base)
        return theta_llama3_scale(th) if self.llama3_scaling else th


CONFIGS = {
    1: AttnConfig("tinyllama-1layer", 32, 4, 64, 1e4, layers=1, prefill=128, decode_steps=32, seed=0),
    2: AttnConfig("llama-3.2-1b", 32, 8, 64, 5e5, layers=16, prefill=2048, decode_steps=256,
                  llama3_scaling=True, seed=1),
    3: AttnConfig("qwen3-8b-shape", 32, 8, 128, 1e6, layers=36, prefill=8192, qk_norm=True,
                  rms_eps=1e-6, bf16_range=True, seed=2),
    4: AttnConfig("llama-3-8b-batched-decode", 32, 8, 128, 5e5, layers=1, batch=64,
                  ctx_range=(512, 8192), block_tokens=16, seed=3),
    5: AttnConfig("70b-class-long-prefill", 64, 8, 128, 5e5, layers=1, prefill=32768, fp16_inputs=True, seed=4),
}


def _bf16_round(a: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 (ties to even) and widen back."""
    u = a.astype(np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)


def rng_for(cfg: AttnConfig, layer: int = 0, stream: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([cfg.seed, layer, stream]))


def gen_qkv(cfg: AttnConfig, n_tok: int, layer: int = 0, stream: int = 0):
    """q [n_tok, n_head, hd], k, v [n_tok, n_head_kv, hd] float32 ~ N(0,1)."""
    g = rng_for(cfg, layer, stream)
    q = g.standard_normal((n_tok, cfg.n_head, cfg.head_dim), dtype=np.float32)
    k = g.standard_normal((n_tok, cfg.n_head_kv, cfg.head_dim), dtype=np.float32)
    v = g.standard_normal((n_tok, cfg.n_head_kv, cfg.head_dim), dtype=np.float32)
    if cfg.bf16_range:
        q, k, v = _bf16_round(q), _bf16_round(k), _bf16_round(v)
    return q, k, v


def gen_norm_weights(cfg: AttnConfig, layer: int = 0):
    """gamma ~ U(0.9, 1.1) for the per-head Q and K RMSNorm, or (None, None)."""
    if not cfg.qk_norm:
        return None, None
    g = rng_for(cfg, layer, 7)
    return (g.uniform(0.9, 1.1, cfg.head_dim).astype(np.float32),
            g.uniform(0.9, 1.1, cfg.head_dim).astype(np.float32))


def gen_ctx_lens(cfg: AttnConfig, batch: int | None = None, rank: int = 0) -> np.ndarray:
    """Context lengths ~ U[lo, hi] (inclusive), one per sequence."""
    g = rng_for(cfg, 0, 100 + rank)
    lo, hi = cfg.ctx_range
    return g.integers(lo, hi + 1, size=batch or cfg.batch).astype(np.int32)


def gen_block_tables(ctx_lens: np.ndarray, block_tokens: int, seed: int, spare: int = 64):
    """A seeded permutation of the pool as physical page order (exercises paging).

    Returns (tables int32 [batch, max_blocks], num_blocks)."""
    need = (ctx_lens.astype(np.int64) + block_tokens - 1) // block_tokens
    num_blocks = int(need.sum()) + spare
    perm = np.random.Generator(np.random.PCG64([seed, 99])).permutation(num_blocks).astype(np.int32)
    max_blocks = int(need.max())
    tables = np.full((len(ctx_lens), max_blocks), -1, np.int32)
    o = 0
    for i, n in enumerate(need):
        tables[i, :n] = perm[o:o + n]
        o += int(n)
    return tables, num_blocks


def shard_longest_first(ctx_lens: np.ndarray, n_ranks: int):
    """Greedy longest-first assignment of sequences to ranks (balances KV bytes)."""
    order = np.argsort(-ctx_lens.astype(np.int64), kind="stable")
    loads = [0] * n_ranks
    owner = [[] for _ in range(n_ranks)]
    for i in order:
        r = loads.index(min(loads))
        owner[r].append(int(i))
        loads[r] += int(ctx_lens[i])
    return [sorted(o) for o in owner]


def gen_sharded_ctx_lens(cfg: AttnConfig, world: int):
    """The batched-decode workload at ``world`` GPUs under weak scaling: ``world`` instances of the seeded
    ``cfg.batch``-sequence workload as ONE set of ``cfg.batch * world`` sequences, dealt to the ranks greedy longest-first.
    Every instance has the same context lengths (each rank fills them with its own K/V data and page order), so the
    deal gives every rank one sequence of each length: per-GPU work -- KV bytes, which is what a decode step costs, not
    sequences -- is the same at every ``world``, which is what weak scaling means.  (Fresh draws per instance differ by
    +-6 % in bytes from one 64-sequence draw to the next, and the one-GPU draw happens to be 13 % lighter than the mean:
    tok/s per GPU would then fall with ``world`` for no reason but the draw.)
    Returns (all context lengths, list of per-rank index lists)."""
    all_ctx = np.tile(gen_ctx_lens(cfg), world)
    return all_ctx, shard_longest_first(all_ctx, world)


def prefill_flops(n_head: int, head_dim: int, n_tok: int, start_pos: int = 0) -> float:
    """4 * hd * n_head * (causal pairs): QK^T and PV, 2 flop per MAC."""
    pairs = n_tok * start_pos + n_tok * (n_tok + 1) / 2
    return 4.0 * head_dim * n_head * pairs


def decode_bytes(ctx_lens, n_head: int, n_head_kv: int, head_dim: int) -> float:
    """K and V read once per KV head (fp16) + q in / out (fp32) + the appended K, V rows."""
    ctx = np.asarray(ctx_lens, dtype=np.int64)
    b = len(ctx)
    return float(ctx.sum() * 2 * n_head_kv * head_dim * 2 + b * n_head * head_dim * 8
                 + b * 2 * n_head_kv * head_dim * 2)
