"""Seeded random shapes through the C ABI against the oracle: head dimension, heads per KV head, page size, RoPE pairing
and rotary width, QK-norm, prompt length, a cached prefix in front of the prompt (prefill at start_pos > 0), then one
batched decode step over the sequence -- every prefill kernel that takes the shape.  The fixed cases elsewhere pin
the configurations of interest; this sweep is for the corners between them."""
import numpy as np
import pytest
import torch

import hippo_leap_b200 as hl
from tests.helpers import assert_parity, oracle_seq

pytestmark = pytest.mark.gpu


def _cases(n, seed, long_prompts=False):
    g = np.random.Generator(np.random.PCG64(seed))
    out = []
    for i in range(n):
        hd = int(g.choice([64, 128, 256], p=[0.4, 0.4, 0.2]))
        n_head_kv = int(g.choice([1, 2, 3, 4]))
        group = int(g.choice([1, 2, 3, 4, 5, 6, 7, 8, 16]))
        bt = int(g.choice([16, 32, 64, 128]))
        rope_mode = int(g.choice([hl.HL_ROPE_INTERLEAVED, hl.HL_ROPE_SPLIT_HALF]))
        rope_dim = hd if g.random() < 0.6 else int(2 * g.integers(1, hd // 2))
        norm = bool(g.random() < 0.5)
        prefix = 0 if g.random() < 0.4 else int(g.integers(1, 400))
        n_tok = int(g.integers(1, 520)) if g.random() < 0.8 else int(g.choice([1, 127, 128, 129, 255, 256, 257, 512]))
        if long_prompts:  # 768 tokens and more: the tcgen05 kernel puts two heads of one KV head into a CTA (even groups)
            n_tok, prefix = int(g.integers(768, 1300)), min(prefix, 200)
            n_head_kv, group = min(n_head_kv, 2), int(g.choice([2, 3, 4, 6, 8]))
        out.append(pytest.param(hd, n_head_kv, group, bt, rope_mode, rope_dim, norm, prefix, n_tok, i + (1000 if long_prompts else 0),
                                id=f"{'L' if long_prompts else ''}{i}-hd{hd}-kv{n_head_kv}x{group}-bt{bt}-rd{rope_dim}-{'n' if norm else 'p'}-{prefix}+{n_tok}"))
    return out


@pytest.mark.parametrize("hd,n_head_kv,group,bt,rope_mode,rope_dim,norm,prefix,n_tok,seed", _cases(28, 20260101) + _cases(8, 20260104, long_prompts=True))
def test_random_shape_prefill_then_decode(hl_ctx, hd, n_head_kv, group, bt, rope_mode, rope_dim, norm, prefix, n_tok, seed):
    n_head = n_head_kv * group
    g = np.random.Generator(np.random.PCG64([seed, 99]))
    theta = hl.theta_table(rope_dim, 1e4)
    hl_ctx.set_rope(theta)
    qw = g.uniform(0.8, 1.2, hd).astype(np.float32) if norm else None
    kw = g.uniform(0.8, 1.2, hd).astype(np.float32) if norm else None
    shape = hl.AttnShape(n_head, n_head_kv, hd, rope_dim, rope_mode, 1e-6,
                         None if qw is None else torch.from_numpy(qw).cuda(), None if kw is None else torch.from_numpy(kw).cuda())
    total = prefix + n_tok + 1
    nb = (total + bt - 1) // bt
    table = torch.from_numpy(g.permutation(nb + 3)[:nb].astype(np.int32)).cuda()
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, nb + 3)
    q = g.standard_normal((total, n_head, hd), dtype=np.float32)
    k = g.standard_normal((total, n_head_kv, hd), dtype=np.float32)
    v = g.standard_normal((total, n_head_kv, hd), dtype=np.float32)
    tq, tk, tv = (torch.from_numpy(x).cuda() for x in (q, k, v))
    kwargs = dict(theta=theta, rope_mode=rope_mode, q_norm_w=qw, k_norm_w=kw)
    try:
        if prefix:
            hl_ctx.kv_append_seq(kv, 0, shape, tk[:prefix], tv[:prefix], 0, table)
        lo, hi = prefix, prefix + n_tok
        hl_ctx.kv_append_seq(kv, 0, shape, tk[lo:hi], tv[lo:hi], lo, table)
        want = oracle_seq(q[lo:hi], k[lo:hi], v[lo:hi], prefix=(k[:lo], v[:lo]) if prefix else None, **kwargs)
        kernels = [0, 1] + ([2] if hd != 256 else []) + ([3] if hd == 128 else [])
        for kernel in kernels:
            hl_ctx.set_tuning(0, kernel)
            try:
                out = hl_ctx.attn_prefill(kv, 0, shape, tq[lo:hi], lo, table)
            finally:
                hl_ctx.set_tuning(0, 0)
            assert_parity(out.cpu().numpy(), want, f"prefill, kernel {kernel}")
        ctx_lens = torch.tensor([total], dtype=torch.int32, device="cuda")
        hl_ctx.kv_append_batch(kv, 0, shape, tk[hi:], tv[hi:], ctx_lens, table.view(1, -1))
        for chunk in (0, 64):
            hl_ctx.set_tuning(chunk, 0)
            try:
                dec = hl_ctx.attn_decode(kv, 0, shape, tq[hi:], ctx_lens, total, table.view(1, -1))
            finally:
                hl_ctx.set_tuning(0, 0)
            assert_parity(dec.cpu().numpy(), oracle_seq(q[hi:], k[hi:], v[hi:], prefix=(k[:hi], v[:hi]), **kwargs),
                          f"decode, chunk {chunk}")
    finally:
        kv.destroy()


def _decode_cases(n, seed):
    g = np.random.Generator(np.random.PCG64(seed))
    out = []
    for i in range(n):
        hd = int(g.choice([64, 128, 256], p=[0.35, 0.5, 0.15]))
        n_head_kv = int(g.choice([1, 2, 4, 8]))
        group = int(g.choice([1, 2, 4, 5, 8, 16]))
        bt = int(g.choice([16, 32, 128]))
        batch = int(g.integers(1, 10))
        hi = int(g.choice([40, 300, 1500]))
        ctxs = [int(x) for x in g.integers(1, hi + 1, batch)]
        chunk = int(g.choice([0, 0, 64, 128, 512]))
        half_io = bool(g.random() < 0.4)
        norm = bool(g.random() < 0.4)
        out.append(pytest.param(hd, n_head_kv, group, bt, ctxs, chunk, half_io, norm, i,
                                id=f"{i}-hd{hd}-kv{n_head_kv}x{group}-bt{bt}-b{batch}-max{max(ctxs)}-c{chunk}-{'f16' if half_io else 'f32'}"))
    return out


@pytest.mark.parametrize("hd,n_head_kv,group,bt,ctxs,chunk,half_io,norm,seed", _decode_cases(24, 20260102))
def test_random_batched_decode_step(hl_ctx, hd, n_head_kv, group, bt, ctxs, chunk, half_io, norm, seed):
    """One decode step of a ragged batch over a shuffled page pool: the new K / V rows appended at each sequence's end,
    then attention over its whole context; float32 or fp16 activations in and out."""
    n_head = n_head_kv * group
    g = np.random.Generator(np.random.PCG64([seed, 7]))
    theta = hl.theta_table(hd, 5e5)
    hl_ctx.set_rope(theta)
    qw = g.uniform(0.8, 1.2, hd).astype(np.float32) if norm else None
    kw = g.uniform(0.8, 1.2, hd).astype(np.float32) if norm else None
    mode = hl.HL_ROPE_SPLIT_HALF if seed % 2 else hl.HL_ROPE_INTERLEAVED
    shape = hl.AttnShape(n_head, n_head_kv, hd, hd, mode, 1e-6,
                         None if qw is None else torch.from_numpy(qw).cuda(), None if kw is None else torch.from_numpy(kw).cuda())
    ctxs = np.asarray(ctxs, np.int32)
    B = len(ctxs)
    need = (ctxs + bt - 1) // bt
    num_blocks = int(need.sum()) + 4
    perm = g.permutation(num_blocks).astype(np.int32)
    tables = np.full((B, int(need.max())), -1, np.int32)
    o = 0
    for i, n in enumerate(need):
        tables[i, :n] = perm[o:o + n]
        o += int(n)
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, num_blocks)
    ttab = torch.from_numpy(tables).cuda()
    dt = np.float16 if half_io else np.float32
    # what the kernels see: activations rounded to the dtype they arrive in
    qn = g.standard_normal((B, n_head, hd), dtype=np.float32).astype(dt)
    kn = g.standard_normal((B, n_head_kv, hd), dtype=np.float32).astype(dt)
    vn = g.standard_normal((B, n_head_kv, hd), dtype=np.float32).astype(dt)
    want = np.zeros((B, n_head, hd), np.float32)
    try:
        for i, c in enumerate(ctxs):
            kp = g.standard_normal((c - 1, n_head_kv, hd), dtype=np.float32)
            vp = g.standard_normal((c - 1, n_head_kv, hd), dtype=np.float32)
            if c > 1:
                hl_ctx.kv_append_seq(kv, 0, shape, torch.from_numpy(kp).cuda(), torch.from_numpy(vp).cuda(), 0,
                                     ttab[i, :need[i]].contiguous())
            want[i] = oracle_seq(qn[i:i + 1].astype(np.float32), kn[i:i + 1].astype(np.float32), vn[i:i + 1].astype(np.float32),
                                 theta=theta, rope_mode=mode, q_norm_w=qw, k_norm_w=kw,
                                 prefix=(kp, vp) if c > 1 else None)[0]
        tctx = torch.from_numpy(ctxs).cuda()
        hl_ctx.set_tuning(chunk, 0)
        try:
            hl_ctx.kv_append_batch(kv, 0, shape, torch.from_numpy(kn).cuda(), torch.from_numpy(vn).cuda(), tctx, ttab)
            out = torch.empty((B, n_head, hd), dtype=torch.float16 if half_io else torch.float32, device="cuda")
            hl_ctx.attn_decode(kv, 0, shape, torch.from_numpy(qn).cuda(), tctx, int(ctxs.max()), ttab, out)
        finally:
            hl_ctx.set_tuning(0, 0)
        tol = dict(max_abs_tol=4e-3, rel_l2_tol=2e-3) if half_io else {}
        assert_parity(out.float().cpu().numpy(), want, "batched decode step", **tol)
    finally:
        kv.destroy()
