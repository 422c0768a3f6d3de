"""Input forms the benchmark configurations use but the small parity cases do not: fp16 Q/K/V handed to the
kernels as fp16 (configuration 5 as specified, the path every head-sharded number runs on), and partial rotary
(rope_dim < head_dim: the dims past rope_dim are copied, not rotated, naive.nim:3200-3201).  Each case compares the
CUDA path, through the C ABI, with the oracle on the same values (inputs rounded to fp16 first where the kernels
receive fp16)."""
import numpy as np
import pytest
import torch

import hippo_leap_b200 as hl
from hippo_leap_b200 import synth
from tests.helpers import assert_parity, oracle_seq

pytestmark = pytest.mark.gpu

KERNELS = [pytest.param(1, id="mma"), pytest.param(2, id="tcgen05"), pytest.param(3, id="tcgen05-pair")]


def _half_round(*xs):
    return tuple(x.astype(np.float16).astype(np.float32) for x in xs)


@pytest.mark.parametrize("S,kernel", [(32768, 2), (32768, 3), (4096, 1)])
def test_config5_fp16_inputs_row_sampled_parity(hl_ctx, S, kernel):
    """Configuration 5 as specified: 64/8 heads, hd 128, theta 5e5, fp16 Q/K/V.  The kernels get fp16 tensors (as
    bench.py hands them over); the oracle gets the same values widened to float32.  48 seeded (token, head) rows."""
    cfg = synth.CONFIGS[5]
    q, k, v = _half_round(*synth.gen_qkv(cfg, S))
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = hl.AttnShape(cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.head_dim, hl.HL_ROPE_SPLIT_HALF, cfg.rms_eps)
    bt = 128
    nb = S // bt
    g = np.random.Generator(np.random.PCG64([5, 43]))
    table = torch.from_numpy(g.permutation(nb + 3)[:nb].astype(np.int32)).cuda()
    kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, nb + 3)
    tq, tk, tv = (torch.from_numpy(x).cuda().half() for x in (q, k, v))
    assert tq.dtype == torch.float16 and torch.equal(tq.float().cpu(), torch.from_numpy(q))
    out = torch.full((S, cfg.n_head, cfg.head_dim), float("nan"), dtype=torch.float16, device="cuda")
    hl_ctx.set_tuning(0, kernel)
    try:
        hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, table)
        hl_ctx.attn_prefill(kv, 0, shape, tq, 0, table, out)
    finally:
        hl_ctx.set_tuning(0, 0)
    rows = np.stack([np.concatenate([[0, 1, S - 1, S // 2, 255, 256], g.integers(0, S, 42)]),
                     g.integers(0, cfg.n_head, 48)], axis=1).astype(np.int32)
    want = oracle_seq(q, k, v, theta=theta, rope_mode=1, rows=rows)
    got = out[torch.from_numpy(rows[:, 0]).long().cuda(), torch.from_numpy(rows[:, 1]).long().cuda()].float().cpu().numpy()
    # fp16 OUTPUT on top of the path's tolerance: half an ulp of values up to ~4 is 2e-3
    assert_parity(got, want, f"config 5 fp16 in/out, S={S}", max_abs_tol=4e-3, rel_l2_tol=2e-3)
    assert torch.isfinite(out).all()
    # float32 output of the same launch stays inside the path's own tolerance
    out32 = torch.empty((S, cfg.n_head, cfg.head_dim), dtype=torch.float32, device="cuda") if S <= 4096 else None
    if out32 is not None:
        hl_ctx.set_tuning(0, kernel)
        try:
            hl_ctx.attn_prefill(kv, 0, shape, tq, 0, table, out32)
        finally:
            hl_ctx.set_tuning(0, 0)
        got32 = out32[torch.from_numpy(rows[:, 0]).long().cuda(), torch.from_numpy(rows[:, 1]).long().cuda()].cpu().numpy()
        assert_parity(got32, want, f"config 5 fp16 in, fp32 out, S={S}")
    kv.destroy()


@pytest.mark.parametrize("hd,n_head,n_head_kv,S,norm", [(128, 8, 2, 300, True), (64, 8, 4, 513, False)])
@pytest.mark.parametrize("kernel", KERNELS)
def test_fp16_inputs_small_full_parity(hl_ctx, hd, n_head, n_head_kv, S, norm, kernel):
    """fp16 Q/K/V views through append, prefill (every kernel) and decode, every row against the oracle."""
    if kernel == 3 and hd != 128:
        pytest.skip("the SM-pair kernel is built for head_dim 128")
    g = np.random.Generator(np.random.PCG64([hd, S, 3]))
    theta = hl.theta_table(hd, 5e5)
    hl_ctx.set_rope(theta)
    qw = g.uniform(0.9, 1.1, hd).astype(np.float32) if norm else None
    kw = g.uniform(0.9, 1.1, hd).astype(np.float32) if norm else None
    shape = hl.AttnShape(n_head, n_head_kv, hd, hd, hl.HL_ROPE_SPLIT_HALF, 1e-6,
                         None if qw is None else torch.from_numpy(qw).cuda(), None if kw is None else torch.from_numpy(kw).cuda())
    q, k, v = _half_round(g.standard_normal((S + 1, n_head, hd), dtype=np.float32),
                          g.standard_normal((S + 1, n_head_kv, hd), dtype=np.float32),
                          g.standard_normal((S + 1, n_head_kv, hd), dtype=np.float32))
    bt = 16
    nb = (S + 1 + bt - 1) // bt
    table = torch.from_numpy(g.permutation(nb).astype(np.int32)).cuda()
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, nb)
    tq, tk, tv = (torch.from_numpy(x).cuda().half() for x in (q, k, v))
    hl_ctx.set_tuning(0, kernel)
    try:
        hl_ctx.kv_append_seq(kv, 0, shape, tk[:S], tv[:S], 0, table)
        out = hl_ctx.attn_prefill(kv, 0, shape, tq[:S], 0, table)
    finally:
        hl_ctx.set_tuning(0, 0)
    want = oracle_seq(q[:S], k[:S], v[:S], theta=theta, rope_mode=1, q_norm_w=qw, k_norm_w=kw)
    assert_parity(out.cpu().numpy(), want, "fp16-input prefill")
    ctx_lens = torch.tensor([S + 1], dtype=torch.int32, device="cuda")
    hl_ctx.kv_append_batch(kv, 0, shape, tk[S:], tv[S:], ctx_lens, table.view(1, -1))
    dec = hl_ctx.attn_decode(kv, 0, shape, tq[S:], ctx_lens, S + 1, table.view(1, -1))
    want_d = oracle_seq(q[S:], k[S:], v[S:], theta=theta, rope_mode=1, q_norm_w=qw, k_norm_w=kw, prefix=(k[:S], v[:S]))
    assert_parity(dec.cpu().numpy(), want_d, "fp16-input decode")
    kv.destroy()


def test_prefill_bcast_with_fp16_inputs_against_the_oracle(hl_ctx):
    """The fused-gather entry point on the input form the head-sharded benchmark uses (fp16 Q, fp16 head-major
    output, extra destinations), against the oracle -- not against another CUDA path."""
    cfg = synth.CONFIGS[5]
    S, bt, n_head, n_head_kv = 1000, 128, 16, 2     # one rank's share of heads at 4 GPUs
    g = np.random.Generator(np.random.PCG64([5, 44]))
    q, k, v = _half_round(g.standard_normal((S, n_head, 128), dtype=np.float32),
                          g.standard_normal((S, n_head_kv, 128), dtype=np.float32),
                          g.standard_normal((S, n_head_kv, 128), dtype=np.float32))
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = hl.AttnShape(n_head, n_head_kv, 128, 128, hl.HL_ROPE_SPLIT_HALF)
    nb = (S + bt - 1) // bt
    table = torch.arange(nb, dtype=torch.int32, device="cuda")
    kv = hl_ctx.kv_create(1, n_head_kv, 128, bt, nb)
    tq, tk, tv = (torch.from_numpy(x).cuda().half() for x in (q, k, v))
    hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, table)
    bufs = [torch.zeros((n_head, S, 128), dtype=torch.float16, device="cuda") for _ in range(3)]
    hl_ctx.attn_prefill_bcast(kv, 0, shape, tq, 0, table, bufs[0].permute(1, 0, 2), [b.data_ptr() for b in bufs[1:]])
    torch.cuda.synchronize()
    want = oracle_seq(q, k, v, theta=theta, rope_mode=1)
    for b in bufs:
        assert_parity(b.permute(1, 0, 2).float().cpu().numpy(), want, "bcast fp16 in/out", max_abs_tol=4e-3, rel_l2_tol=2e-3)
    kv.destroy()


@pytest.mark.parametrize("hd,rope_dim", [(128, 64), (64, 32), (128, 96), (128, 78), (256, 64)])  # 78 of 128: Nemotron-H (tests/integration_nemotron.nim:33)
@pytest.mark.parametrize("rope_mode", [hl.HL_ROPE_INTERLEAVED, hl.HL_ROPE_SPLIT_HALF], ids=["interleaved", "split-half"])
@pytest.mark.parametrize("kernel", KERNELS)
def test_partial_rotary(hl_ctx, hd, rope_dim, rope_mode, kernel):
    """rope_dim < head_dim: only the first rope_dim dims of Q and K are rotated (pairs (2i, 2i+1) or (i, i + rope_dim/2)),
    the rest pass through (naive.nim:3200-3201) -- for append, prefill (every kernel; the tcgen05 kernels take their
    general query prologue here) and decode."""
    if kernel == 3 and hd != 128:
        pytest.skip("the SM-pair kernel is built for head_dim 128")
    if kernel == 2 and hd == 256:
        pytest.skip("head_dim 256 runs on the warp-MMA kernel")
    n_head, n_head_kv, S, bt = 8, 2, 333, 16
    g = np.random.Generator(np.random.PCG64([hd, rope_dim, rope_mode]))
    theta = hl.theta_table(rope_dim, 1e4)          # rope_dim / 2 frequencies
    assert theta.shape[0] == rope_dim // 2
    hl_ctx.set_rope(theta)
    qw = g.uniform(0.9, 1.1, hd).astype(np.float32)
    kw = g.uniform(0.9, 1.1, hd).astype(np.float32)
    shape = hl.AttnShape(n_head, n_head_kv, hd, rope_dim, rope_mode, 1e-6, torch.from_numpy(qw).cuda(),
                         torch.from_numpy(kw).cuda())
    q = g.standard_normal((S + 1, n_head, hd), dtype=np.float32)
    k = g.standard_normal((S + 1, n_head_kv, hd), dtype=np.float32)
    v = g.standard_normal((S + 1, n_head_kv, hd), dtype=np.float32)
    nb = (S + 1 + bt - 1) // bt
    table = torch.from_numpy(g.permutation(nb).astype(np.int32)).cuda()
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, nb)
    tq, tk, tv = (torch.from_numpy(x).cuda() for x in (q, k, v))
    hl_ctx.set_tuning(0, kernel)
    try:
        hl_ctx.kv_append_seq(kv, 0, shape, tk[:S], tv[:S], 0, table)
        out = hl_ctx.attn_prefill(kv, 0, shape, tq[:S], 0, table)
    finally:
        hl_ctx.set_tuning(0, 0)
    kwargs = dict(theta=theta, rope_mode=rope_mode, q_norm_w=qw, k_norm_w=kw)
    assert_parity(out.cpu().numpy(), oracle_seq(q[:S], k[:S], v[:S], **kwargs), "partial-rotary prefill")
    # against the oracle that rounds K (after norm and RoPE) and V to fp16 like the cache does: a rotated tail or a
    # missed pair would show here at 1e-1; what is left is the fp16 rounding of Q and P inside the kernels
    assert_parity(out.cpu().numpy(), oracle_seq(q[:S], k[:S], v[:S], kv_fp16=True, **kwargs),
                  "partial-rotary prefill vs fp16-KV oracle", 1.5e-3, 6e-4)
    ctx_lens = torch.tensor([S + 1], dtype=torch.int32, device="cuda")
    hl_ctx.kv_append_batch(kv, 0, shape, tk[S:], tv[S:], ctx_lens, table.view(1, -1))
    dec = hl_ctx.attn_decode(kv, 0, shape, tq[S:], ctx_lens, S + 1, table.view(1, -1))
    assert_parity(dec.cpu().numpy(), oracle_seq(q[S:], k[S:], v[S:], prefix=(k[:S], v[:S]), **kwargs), "partial-rotary decode")
    # the cached K rows: dims >= rope_dim are the normed input, bit for bit what a full-width fp16 rounding gives
    kp, _, nbytes = kv.layer_ptrs(0)

    class _Pool:  # zero-copy view of the layer's K pool through the CUDA array interface
        __cuda_array_interface__ = {"shape": (nbytes // 2,), "typestr": "<f2", "data": (kp, False), "version": 2}

    pool = torch.as_tensor(_Pool(), device="cuda").view(nb, n_head_kv, bt, hd)
    tok = 37
    row = pool[int(table[tok // bt]), 1, tok % bt].float().cpu().numpy()
    x = k[tok, 1]
    normed = x * (1.0 / np.sqrt(np.float32((x * x).sum() / hd + 1e-6))) * kw
    assert np.abs(row[rope_dim:] - normed[rope_dim:].astype(np.float16).astype(np.float32)).max() <= 1e-3
    assert np.abs(row[:rope_dim] - normed[:rope_dim]).max() > 1e-2     # and the head of the row did rotate
    kv.destroy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("kernel", [pytest.param(1, id="mma"), pytest.param(2, id="tcgen05")])
def test_head_major_query_and_output_views(hl_ctx, dtype, kernel):
    """Q, K, V and the output held head-major ([heads][tokens][head_dim]: the token stride is SMALLER than the head
    stride) and passed as [tokens][heads][head_dim] views -- the layout the head-sharded runners write -- through append,
    prefill (whichever query prologue the view gets: staged by TMA when the copy engine can describe it, registers
    otherwise) and decode, against the oracle."""
    hd, n_head, n_head_kv, S, bt = 128, 8, 2, 700, 16
    g = np.random.Generator(np.random.PCG64([S, 17]))
    theta = hl.theta_table(hd, 5e5)
    hl_ctx.set_rope(theta)
    shape = hl.AttnShape(n_head, n_head_kv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    q, k, v = (g.standard_normal((S + 1, h_, hd), dtype=np.float32) for h_ in (n_head, n_head_kv, n_head_kv))
    if dtype == torch.float16:
        q, k, v = _half_round(q, k, v)
    nb = (S + 1 + bt - 1) // bt
    table = torch.from_numpy(g.permutation(nb).astype(np.int32)).cuda()
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, nb)
    # head-major storage, token-major views
    hq, hk, hv = (torch.from_numpy(x).cuda().to(dtype).permute(1, 0, 2).contiguous() for x in (q, k, v))
    tq, tk, tv = (x.permute(1, 0, 2) for x in (hq, hk, hv))
    assert tq.stride(0) < tq.stride(1)
    out_hm = torch.full((n_head, S, hd), float("nan"), dtype=torch.float32, device="cuda")
    hl_ctx.set_tuning(0, kernel)
    try:
        hl_ctx.kv_append_seq(kv, 0, shape, tk[:S], tv[:S], 0, table)
        hl_ctx.attn_prefill(kv, 0, shape, tq[:S], 0, table, out_hm.permute(1, 0, 2))
    finally:
        hl_ctx.set_tuning(0, 0)
    want = oracle_seq(q[:S], k[:S], v[:S], theta=theta, rope_mode=1)
    assert_parity(out_hm.permute(1, 0, 2).cpu().numpy(), want, "head-major views, prefill")
    ctx_lens = torch.tensor([S + 1], dtype=torch.int32, device="cuda")
    hl_ctx.kv_append_batch(kv, 0, shape, tk[S:], tv[S:], ctx_lens, table.view(1, -1))
    dec = hl_ctx.attn_decode(kv, 0, shape, tq[S:], ctx_lens, S + 1, table.view(1, -1))
    want_d = oracle_seq(q[S:], k[S:], v[S:], theta=theta, rope_mode=1, prefix=(k[:S], v[:S]))
    assert_parity(dec.cpu().numpy(), want_d, "head-major views, decode")
    kv.destroy()
