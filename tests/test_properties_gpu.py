"""GPU checks at the benchmark sizes through properties that do not need a full CPU run:
row-sampled oracle parity, constant-V checksum, paging invariance, chunked = unchunked prefill,
prefill/decode cross-consistency, reference `[dim, S]` layout views, fp16 output."""
import numpy as np
import pytest
import torch

import hippo_leap_b200 as hl
from hippo_leap_b200 import synth
from tests.helpers import assert_parity, oracle_seq

pytestmark = pytest.mark.gpu


def _upload(*xs):
    return tuple(torch.from_numpy(x).cuda() for x in xs)


def _shape_for(cfg, rope_mode, qw=None, kw=None):
    return hl.AttnShape(cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.head_dim, rope_mode, cfg.rms_eps,
                        None if qw is None else torch.from_numpy(qw).cuda(),
                        None if kw is None else torch.from_numpy(kw).cuda())


@pytest.mark.parametrize("ci,S,kernel", [(2, 2048, 1), (2, 2048, 2), (3, 8192, 2), (3, 8192, 3), (5, 32768, 2), (5, 32768, 3), (5, 4096, 1)])
def test_prefill_row_sampled_parity_at_config_sizes(hl_ctx, ci, S, kernel):
    """Configs 2, 3 and 5 at their full prompt lengths (one layer): 48 seeded (token, head) rows are
    checked against the oracle, which computes exactly those rows."""
    cfg = synth.CONFIGS[ci]
    q, k, v = synth.gen_qkv(cfg, S)
    qw, kw = synth.gen_norm_weights(cfg)
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = _shape_for(cfg, hl.HL_ROPE_INTERLEAVED, qw, kw)
    bt = 16 if ci == 2 else 128
    nb = (S + bt - 1) // bt
    g = np.random.Generator(np.random.PCG64([ci, 42]))
    table = g.permutation(nb + 5)[:nb].astype(np.int32)
    kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, nb + 5)
    tq, tk, tv, tt = _upload(q, k, v, table)
    hl_ctx.set_tuning(0, kernel)
    hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, tt)
    out = hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt)
    hl_ctx.set_tuning(0, 0)
    rows = np.stack([np.concatenate([[0, 1, S - 1, S // 2], g.integers(0, S, 44)]),
                     g.integers(0, cfg.n_head, 48)], axis=1).astype(np.int32)
    want = oracle_seq(q, k, v, theta=theta, rope_mode=0, q_norm_w=qw, k_norm_w=kw, eps=cfg.rms_eps, rows=rows)
    got = out[torch.from_numpy(rows[:, 0]).long().cuda(), torch.from_numpy(rows[:, 1]).long().cuda()].cpu().numpy()
    assert_parity(got, want, f"config {ci} S={S} sampled rows")
    assert torch.isfinite(out).all()
    kv.destroy()


@pytest.mark.parametrize("kernel", [1, 2], ids=["mma", "tcgen05"])
def test_constant_v_checksum_and_paging_invariance(hl_ctx, kernel):
    """softmax rows sum to one: with V == 0.75 everywhere every output is 0.75 (exact in fp16);
    and the physical page order must not change a single bit of the result."""
    cfg = synth.CONFIGS[5]
    S, bt = 4096 + 77, 16
    q, k, v = synth.gen_qkv(cfg, S)
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = _shape_for(cfg, hl.HL_ROPE_SPLIT_HALF)
    nb = (S + bt - 1) // bt
    tq, tk, tv = _upload(q, k, v)
    hl_ctx.set_tuning(0, kernel)
    outs = []
    for seed in (1, 2):
        table = np.random.Generator(np.random.PCG64(seed)).permutation(nb + 9)[:nb].astype(np.int32)
        tt, = _upload(table)
        kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, nb + 9)
        hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, tt)
        outs.append(hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt).clone())
        if seed == 2:
            vc = torch.full_like(tv, 0.75)
            hl_ctx.kv_append_seq(kv, 0, shape, tk, vc, 0, tt)
            oc = hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt)
            assert float((oc - 0.75).abs().max()) < 2e-4
        kv.destroy()
    hl_ctx.set_tuning(0, 0)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("kernel", [1, 2], ids=["mma", "tcgen05"])
def test_chunked_prefill_equals_unchunked(hl_ctx, kernel):
    """start_pos != 0: appending and attending in two chunks gives the rows of one pass."""
    cfg = synth.CONFIGS[3]
    S, S1, bt = 1000, 389, 16
    q, k, v = synth.gen_qkv(cfg, S)
    qw, kw = synth.gen_norm_weights(cfg)
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = _shape_for(cfg, hl.HL_ROPE_SPLIT_HALF, qw, kw)
    nb = (S + bt - 1) // bt
    tq, tk, tv = _upload(q, k, v)
    tt = torch.arange(nb, dtype=torch.int32, device="cuda").flip(0).contiguous()
    hl_ctx.set_tuning(0, kernel)
    kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, nb)
    hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, tt)
    full = hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt).clone()
    kv2 = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, nb)
    hl_ctx.kv_append_seq(kv2, 0, shape, tk[:S1], tv[:S1], 0, tt)
    a = hl_ctx.attn_prefill(kv2, 0, shape, tq[:S1], 0, tt).clone()
    hl_ctx.kv_append_seq(kv2, 0, shape, tk[S1:], tv[S1:], S1, tt)
    b = hl_ctx.attn_prefill(kv2, 0, shape, tq[S1:], S1, tt).clone()
    hl_ctx.set_tuning(0, 0)
    # same keys, same arithmetic per row up to the tile order of the online softmax
    assert float((torch.cat([a, b]) - full).abs().max()) < 5e-4
    want = oracle_seq(q[S1:S1 + 4], k[S1:S1 + 4], v[S1:S1 + 4], theta=theta, rope_mode=1, q_norm_w=qw, k_norm_w=kw,
                      eps=cfg.rms_eps, prefix=(k[:S1], v[:S1]))
    assert_parity(b[:4].cpu().numpy(), want, "second chunk vs oracle")
    kv.destroy()
    kv2.destroy()


def test_decode_matches_prefill_last_row_at_long_context(hl_ctx):
    """Cross-kernel consistency at 32k keys: the decode kernel on the last token reproduces the
    prefill kernel's last row, and both match the oracle row."""
    cfg = synth.CONFIGS[5]
    S, bt = 32768, 16
    q, k, v = synth.gen_qkv(cfg, S)
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = _shape_for(cfg, hl.HL_ROPE_SPLIT_HALF)
    nb = S // bt
    tq, tk, tv = _upload(q, k, v)
    tt = torch.randperm(nb, device="cuda").to(torch.int32)
    kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, nb)
    hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, tt)
    pre = hl_ctx.attn_prefill(kv, 0, shape, tq[S - 256:], S - 256, tt)
    ctx_lens = torch.tensor([S], dtype=torch.int32, device="cuda")
    dec = hl_ctx.attn_decode(kv, 0, shape, tq[S - 1:], ctx_lens, S, tt.view(1, -1))
    assert float((dec[0] - pre[-1]).abs().max()) < 3e-4
    rows = np.array([[S - 1, h] for h in (0, 17, 63)], np.int32)
    want = oracle_seq(q, k, v, theta=theta, rope_mode=1, rows=rows)
    assert_parity(dec[0, [0, 17, 63]].cpu().numpy(), want, "decode at 32k")
    kv.destroy()


def test_reference_dim_major_layout_and_fp16_output(hl_ctx):
    """Inputs and outputs in the reference's `[dim, S]` token-fastest layout (naive.nim:2984-2990),
    and fp16 output, give the same numbers as token-major fp32."""
    cfg = synth.CONFIGS[1]
    S, bt = 128, 16
    q, k, v = synth.gen_qkv(cfg, S)
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = _shape_for(cfg, hl.HL_ROPE_SPLIT_HALF)
    tq, tk, tv = _upload(q, k, v)
    tt = torch.arange(S // bt, dtype=torch.int32, device="cuda")
    kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, S // bt)
    hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, tt)
    base = hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt).clone()
    # [dim, S] buffers viewed as [S, heads, hd]
    q_ds = tq.permute(1, 2, 0).contiguous()  # [H, hd, S] == [qDim, S]
    k_ds = tk.permute(1, 2, 0).contiguous()
    v_ds = tv.permute(1, 2, 0).contiguous()
    out_ds = torch.empty_like(q_ds)
    kv2 = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, S // bt)
    hl_ctx.kv_append_seq(kv2, 0, shape, k_ds.permute(2, 0, 1), v_ds.permute(2, 0, 1), 0, tt)
    for kernel in (1, 2):
        hl_ctx.set_tuning(0, kernel)
        hl_ctx.attn_prefill(kv2, 0, shape, q_ds.permute(2, 0, 1), 0, tt, out_ds.permute(2, 0, 1))
        assert float((out_ds.permute(2, 0, 1) - base).abs().max()) < 6e-4
        o16 = torch.empty((S, cfg.n_head, cfg.head_dim), dtype=torch.float16, device="cuda")
        hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt, o16)
        assert float((o16.float() - base).abs().max()) < 4e-3
    hl_ctx.set_tuning(0, 0)
    want = oracle_seq(q, k, v, theta=theta, rope_mode=1)
    assert_parity(out_ds.permute(2, 0, 1).cpu().numpy(), want, "dim-major layout")
    kv.destroy()
    kv2.destroy()


def test_config4_batched_decode_sampled_parity(hl_ctx):
    """Config 4 at full size (64 sequences, ctx ~U[512, 8192], permuted 16-token pages): every
    sequence's output row of 3 heads is checked against the oracle."""
    cfg = synth.CONFIGS[4]
    ctx_lens = synth.gen_ctx_lens(cfg)
    tables, num_blocks = synth.gen_block_tables(ctx_lens, cfg.block_tokens, cfg.seed)
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = _shape_for(cfg, hl.HL_ROPE_SPLIT_HALF)
    kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, cfg.block_tokens, num_blocks)
    ttab, tctx = _upload(tables, ctx_lens)
    B = len(ctx_lens)
    g = synth.rng_for(cfg, 0, 5)
    qn = g.standard_normal((B, cfg.n_head, cfg.head_dim), dtype=np.float32)
    prefixes = []
    for i, c in enumerate(ctx_lens):
        kk = g.standard_normal((int(c), cfg.n_head_kv, cfg.head_dim), dtype=np.float32)
        vv = g.standard_normal((int(c), cfg.n_head_kv, cfg.head_dim), dtype=np.float32)
        prefixes.append((kk, vv))
        nb = (int(c) + cfg.block_tokens - 1) // cfg.block_tokens
        tk, tv = _upload(kk[:-1], vv[:-1])
        hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, ttab[i, :nb].contiguous())
    kn = np.stack([p[0][-1] for p in prefixes])
    vn = np.stack([p[1][-1] for p in prefixes])
    tqn, tkn, tvn = _upload(qn, kn, vn)
    hl_ctx.kv_append_batch(kv, 0, shape, tkn, tvn, tctx, ttab)
    out = hl_ctx.attn_decode(kv, 0, shape, tqn, tctx, int(ctx_lens.max()), ttab).cpu().numpy()
    heads = [0, 13, 31]
    rows = np.array([[0, h] for h in heads], np.int32)
    for i in range(B):
        kk, vv = prefixes[i]
        want = oracle_seq(qn[i:i + 1], kk[-1:], vv[-1:], theta=theta, rope_mode=1, rows=rows, prefix=(kk[:-1], vv[:-1]))
        assert_parity(out[i, heads], want, f"config 4 sequence {i} (ctx {ctx_lens[i]})")
    kv.destroy()


def test_head_sharded_prefill_runner_single_rank_equals_plain_prefill(hl_ctx):
    """The chunked, overlapped head-sharded runner (world size 1 here: the gather is a copy) returns the
    rows of one plain prefill call, in its [chunk][head][row][dim] layout."""
    from hippo_leap_b200 import sharding
    cfg = synth.CONFIGS[3]
    S, bt = 2048, 128
    q, k, v = synth.gen_qkv(cfg, S)
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = _shape_for(cfg, hl.HL_ROPE_SPLIT_HALF)
    tq, tk, tv = _upload(q, k, v)
    tt = torch.arange(S // bt, dtype=torch.int32, device="cuda")
    kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, S // bt)
    hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, tt)
    plain = hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt)
    runner = sharding.HeadShardedPrefill(hl_ctx, kv, shape, S, 4, tq.device, world=1)
    full = runner.run(tq, tt)  # [4, H, 512, hd] fp16
    torch.cuda.synchronize()
    got = full.permute(0, 2, 1, 3).reshape(S, cfg.n_head, cfg.head_dim).float()
    assert float((got - plain).abs().max()) < 4e-3  # fp16 output rounding only
    rows = np.array([[5, 0], [700, 9], [2047, 31]], np.int32)
    want = oracle_seq(q, k, v, theta=theta, rope_mode=1, rows=rows)
    assert_parity(got[[5, 700, 2047], [0, 9, 31]].cpu().numpy(), want, "head-sharded runner rows",
                  max_abs_tol=4e-3, rel_l2_tol=2e-3)  # fp16 OUTPUT variant: its own rounding on top of the path's
    kv.destroy()


def test_prefill_bcast_writes_identical_copies_to_every_destination(hl_ctx):
    """The fused gather path on one GPU: three extra destinations (local buffers standing in for peers'
    mapped memory) must receive bit-identical copies of the output, for both output dtypes."""
    cfg = synth.CONFIGS[3]
    S, bt = 700, 16
    q, k, v = synth.gen_qkv(cfg, S)
    qw, kw = synth.gen_norm_weights(cfg)
    hl_ctx.set_rope(cfg.theta())
    shape = _shape_for(cfg, hl.HL_ROPE_SPLIT_HALF, qw, kw)
    tq, tk, tv = _upload(q, k, v)
    nb = (S + bt - 1) // bt
    tt = torch.randperm(nb, device="cuda").to(torch.int32)
    kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, nb)
    hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, tt)
    want = hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt)
    for dtype in (torch.float16, torch.float32):
        bufs = [torch.zeros((cfg.n_head, S, cfg.head_dim), dtype=dtype, device="cuda") for _ in range(4)]
        hl_ctx.attn_prefill_bcast(kv, 0, shape, tq, 0, tt, bufs[0].permute(1, 0, 2), [b.data_ptr() for b in bufs[1:]])
        torch.cuda.synchronize()
        for b in bufs[1:]:
            assert torch.equal(b, bufs[0])
        tol = 4e-3 if dtype == torch.float16 else 3e-4  # tcgen05 path vs the default path, plus fp16 rounding
        assert float((bufs[0].permute(1, 0, 2).float() - want).abs().max()) < tol
    with pytest.raises(hl.HlError):
        hl_ctx.attn_prefill_bcast(kv, 0, shape, tq, 0, tt, bufs[0].permute(1, 0, 2), [1] * 8)
    kv.destroy()
