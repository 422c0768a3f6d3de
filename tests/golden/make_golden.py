"""Generates tests/golden/attn_golden.npz: small seeded inputs and the oracle's outputs for them.

The reference (Nim) cannot run where this repository is developed, so these vectors are produced by
the CPU oracle (oracle/tensor_ref.c), not by the reference itself: they pin the oracle against
regressions (compiler flags, refactors) and give the CUDA path fixed numbers to match.
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

CASES = [
    # name, S, n_head, n_head_kv, hd, base, rope_mode, qk_norm, decode_steps
    ("tiny_interleaved", 24, 4, 2, 64, 1e4, 0, False, 3),
    ("tiny_split_half", 24, 4, 2, 64, 1e4, 1, False, 3),
    ("hd128_norm", 20, 4, 2, 128, 1e6, 1, True, 2),
    ("single_token", 1, 4, 4, 64, 5e5, 0, False, 2),
]


def main():
    out = {}
    for ci, (name, S, H, Hkv, hd, base, mode, norm, steps) in enumerate(CASES):
        g = np.random.Generator(np.random.PCG64([2024, ci]))
        T = S + steps
        q = g.standard_normal((T, H, hd), dtype=np.float32)
        k = g.standard_normal((T, Hkv, hd), dtype=np.float32)
        v = g.standard_normal((T, Hkv, hd), dtype=np.float32)
        qw = g.uniform(0.9, 1.1, hd).astype(np.float32) if norm else None
        kw = g.uniform(0.9, 1.1, hd).astype(np.float32) if norm else None
        theta = oracle.theta_table(hd, base)
        for tag, fp16 in (("f32", False), ("kv16", True)):
            cache = oracle.SeqCache(T, Hkv, hd)
            outs = [oracle.attn_forward(q[:S], k[:S], v[:S], cache, theta=theta, rope_mode=mode, q_norm_w=qw,
                                        k_norm_w=kw, eps=1e-6, kv_fp16=fp16)]
            for t in range(S, T):
                outs.append(oracle.attn_forward(q[t:t + 1], k[t:t + 1], v[t:t + 1], cache, theta=theta,
                                                rope_mode=mode, q_norm_w=qw, k_norm_w=kw, eps=1e-6, kv_fp16=fp16))
            out[f"{name}/out_{tag}"] = np.concatenate(outs)
            if not fp16:
                out[f"{name}/k_cache"] = cache.k.copy()
        out[f"{name}/q"], out[f"{name}/k"], out[f"{name}/v"] = q, k, v
        out[f"{name}/theta"] = theta
        if norm:
            out[f"{name}/qw"], out[f"{name}/kw"] = qw, kw
        out[f"{name}/meta"] = np.array([S, H, Hkv, hd, mode, int(norm), steps], np.int64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
