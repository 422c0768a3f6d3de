"""Shared helpers of the parity tests: metrics, oracle drivers, paged-cache set-up."""
from __future__ import annotations

import numpy as np

import oracle

# Tolerances of the path (fp16 KV cache, fp32 accumulation) against the fp32 CPU oracle.
MAX_ABS = 2e-3
REL_L2 = 1e-3


def max_abs(a, b) -> float:
    return float(np.max(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64))))


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def assert_parity(got, want, what="", max_abs_tol=MAX_ABS, rel_l2_tol=REL_L2):
    ma, rl = max_abs(got, want), rel_l2(got, want)
    assert np.isfinite(np.asarray(got)).all(), f"{what}: non-finite output"
    assert ma <= max_abs_tol and rl <= rel_l2_tol, (
        f"{what}: max-abs {ma:.3e} (limit {max_abs_tol:.1e}), rel-L2 {rl:.3e} (limit {rel_l2_tol:.1e})")
    return ma, rl


def oracle_seq(q, k, v, *, theta, rope_mode, q_norm_w=None, k_norm_w=None, eps=1e-6,
               kv_fp16=False, rows=None, prefix=None, n_threads=0):
    """Run the oracle on one sequence.  prefix = (k_prev, v_prev) raw rows already in the cache
    (they are appended first, attention rows for them are not computed)."""
    n_prev = 0 if prefix is None else prefix[0].shape[0]
    cache = oracle.SeqCache(n_prev + q.shape[0], k.shape[1], k.shape[2])
    if n_prev:
        qz = np.zeros((n_prev, q.shape[1], q.shape[2]), np.float32)
        oracle.attn_forward(qz, prefix[0], prefix[1], cache, theta=theta, rope_mode=rope_mode,
                            k_norm_w=k_norm_w, eps=eps, kv_fp16=kv_fp16, rows=[[0, 0]], n_threads=1)
    return oracle.attn_forward(q, k, v, cache, theta=theta, rope_mode=rope_mode, q_norm_w=q_norm_w,
                               k_norm_w=k_norm_w, eps=eps, kv_fp16=kv_fp16, rows=rows,
                               n_threads=n_threads)


def permuted_table(n_blocks_needed: int, num_blocks: int, seed: int) -> np.ndarray:
    perm = np.random.Generator(np.random.PCG64([seed, 5])).permutation(num_blocks)
    return perm[:n_blocks_needed].astype(np.int32)
