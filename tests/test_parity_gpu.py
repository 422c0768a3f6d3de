"""GPU parity of the CUDA path (through the C ABI) against the CPU oracle, on small seeded cases."""
import numpy as np
import pytest
import torch

import hippo_leap_b200 as hl
from tests.helpers import assert_parity, oracle_seq, permuted_table

pytestmark = pytest.mark.gpu


def _setup(hl_ctx, n_head, n_head_kv, hd, S_total, bt, rope_mode, norm, seed, base=1e4):
    g = np.random.Generator(np.random.PCG64(seed))
    theta = hl.theta_table(hd, base)
    hl_ctx.set_rope(theta)
    qw = kw = None
    if norm:
        qw = g.uniform(0.9, 1.1, hd).astype(np.float32)
        kw = g.uniform(0.9, 1.1, hd).astype(np.float32)
    shape = hl.AttnShape(n_head, n_head_kv, hd, hd, rope_mode, 1e-6,
                         None if qw is None else torch.from_numpy(qw).cuda(),
                         None if kw is None else torch.from_numpy(kw).cuda())
    n_blocks = (S_total + bt - 1) // bt
    num_blocks = n_blocks + 7
    table = permuted_table(n_blocks, num_blocks, seed)
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, num_blocks)
    return g, theta, qw, kw, shape, kv, table


@pytest.mark.parametrize("hd,n_head,n_head_kv,S,bt,rope_mode,norm", [
    (64, 32, 4, 128, 16, hl.HL_ROPE_INTERLEAVED, False),   # config 1 prefill
    (64, 32, 4, 128, 16, hl.HL_ROPE_SPLIT_HALF, False),
    (128, 8, 2, 200, 16, hl.HL_ROPE_SPLIT_HALF, True),
    (128, 4, 4, 1, 16, hl.HL_ROPE_INTERLEAVED, False),
    (64, 4, 1, 17, 32, hl.HL_ROPE_INTERLEAVED, True),
    (128, 8, 1, 257, 64, hl.HL_ROPE_SPLIT_HALF, False),
    (128, 4, 2, 513, 128, hl.HL_ROPE_INTERLEAVED, False),
    (128, 4, 2, 640, 128, hl.HL_ROPE_SPLIT_HALF, True),
    (128, 10, 2, 300, 16, hl.HL_ROPE_SPLIT_HALF, False),    # group of 5 query heads per KV head (Nemotron-H: 40 / 8)
    (64, 14, 2, 270, 16, hl.HL_ROPE_INTERLEAVED, True),     # group of 7 (28 / 4 models)
    (256, 8, 1, 300, 16, hl.HL_ROPE_SPLIT_HALF, True),      # head_dim 256, 16 / 2 heads (the reference's qwen35moe
    (256, 4, 2, 70, 32, hl.HL_ROPE_INTERLEAVED, False),     # attention layers, tests/integration_qwen36moe.nim:25-27)
    (64, 8, 2, 300, 16, hl.HL_ROPE_SPLIT_HALF, False),
])
@pytest.mark.parametrize("kernel", [1, 2, 3], ids=["mma", "tcgen05", "tcgen05-pair"])
def test_prefill_parity(hl_ctx, hd, n_head, n_head_kv, S, bt, rope_mode, norm, kernel):
    if kernel == 3 and hd != 128:
        pytest.skip("the SM-pair kernel is built for head_dim 128")
    if kernel == 2 and hd == 256:
        pytest.skip("head_dim 256 runs on the warp-MMA kernel (the tcgen05 kernels are built for 64 and 128)")
    g, theta, qw, kw, shape, kv, table = _setup(hl_ctx, n_head, n_head_kv, hd, S, bt, rope_mode, norm, 11)
    q = g.standard_normal((S, n_head, hd), dtype=np.float32)
    k = g.standard_normal((S, n_head_kv, hd), dtype=np.float32)
    v = g.standard_normal((S, n_head_kv, hd), dtype=np.float32)
    tq, tk, tv = (torch.from_numpy(x).cuda() for x in (q, k, v))
    tt = torch.from_numpy(table).cuda()
    hl_ctx.set_tuning(0, kernel)
    hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, tt)
    out = hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt)
    got = out.cpu().numpy()
    # host-buffer form (append + prefill, host in / host out) equals the device form
    out_h = torch.full((S, n_head, hd), float("nan"))
    hl_ctx.prefill_host(kv, 0, shape, torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v), 0, tt, out_h)
    assert np.array_equal(out_h.numpy(), got), "prefill_host differs from the device form"
    hl_ctx.set_tuning(0, 0)
    want = oracle_seq(q, k, v, theta=theta, rope_mode=rope_mode, q_norm_w=qw, k_norm_w=kw)
    want16 = oracle_seq(q, k, v, theta=theta, rope_mode=rope_mode, q_norm_w=qw, k_norm_w=kw, kv_fp16=True)
    assert_parity(got, want, "prefill vs fp32 oracle")
    assert_parity(got, want16, "prefill vs fp16-KV oracle", 1e-3, 6e-4)
    kv.destroy()


@pytest.mark.parametrize("hd,n_head,n_head_kv,bt,rope_mode,norm,ctxs,chunk", [
    (64, 32, 4, 16, hl.HL_ROPE_INTERLEAVED, False, [129], 0),          # config 1 first decode step
    (128, 32, 8, 16, hl.HL_ROPE_SPLIT_HALF, False, [1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256, 257, 700], 0),
    (128, 32, 8, 16, hl.HL_ROPE_SPLIT_HALF, True, [300, 1, 1000, 64], 64),
    (128, 8, 8, 32, hl.HL_ROPE_INTERLEAVED, False, [513, 77], 128),
    (64, 16, 1, 16, hl.HL_ROPE_SPLIT_HALF, True, [90, 200, 333], 0),
    (128, 10, 2, 16, hl.HL_ROPE_SPLIT_HALF, False, [1, 31, 260, 700], 0),    # group of 5
    (64, 14, 2, 16, hl.HL_ROPE_INTERLEAVED, True, [65, 500], 64),            # group of 7
    (128, 12, 1, 16, hl.HL_ROPE_SPLIT_HALF, False, [130], 0),                # group of 12
    (256, 16, 2, 16, hl.HL_ROPE_SPLIT_HALF, True, [1, 64, 65, 300, 1000], 0),   # head_dim 256 (qwen35moe: 16 / 2 heads)
    (256, 4, 4, 32, hl.HL_ROPE_INTERLEAVED, False, [200, 33], 64),
])
def test_decode_parity(hl_ctx, hd, n_head, n_head_kv, bt, rope_mode, norm, ctxs, chunk):
    ctxs = np.asarray(ctxs, np.int32)
    B = len(ctxs)
    g, theta, qw, kw, shape, _kv, _ = _setup(hl_ctx, n_head, n_head_kv, hd, 16, bt, rope_mode, norm, 23)
    _kv.destroy()
    need = (ctxs + bt - 1) // bt
    num_blocks = int(need.sum()) + 5
    perm = g.permutation(num_blocks).astype(np.int32)
    tables = np.full((B, int(need.max())), -1, np.int32)
    o = 0
    for i, n in enumerate(need):
        tables[i, :n] = perm[o:o + n]
        o += int(n)
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, num_blocks)
    ttab = torch.from_numpy(tables).cuda()
    want = np.zeros((B, n_head, hd), np.float32)
    want16 = np.zeros_like(want)
    qn = g.standard_normal((B, n_head, hd), dtype=np.float32)
    kn = g.standard_normal((B, n_head_kv, hd), dtype=np.float32)
    vn = g.standard_normal((B, n_head_kv, hd), dtype=np.float32)
    for i, c in enumerate(ctxs):
        kp = g.standard_normal((c - 1, n_head_kv, hd), dtype=np.float32)
        vp = g.standard_normal((c - 1, n_head_kv, hd), dtype=np.float32)
        if c > 1:
            hl_ctx.kv_append_seq(kv, 0, shape, torch.from_numpy(kp).cuda(), torch.from_numpy(vp).cuda(), 0,
                                 ttab[i, :need[i]].contiguous())
        for fp16, dst in ((False, want), (True, want16)):
            dst[i] = oracle_seq(qn[i:i + 1], kn[i:i + 1], vn[i:i + 1], theta=theta, rope_mode=rope_mode,
                                q_norm_w=qw, k_norm_w=kw, kv_fp16=fp16,
                                prefix=(kp, vp) if c > 1 else None)[0]
    tctx = torch.from_numpy(ctxs).cuda()
    hl_ctx.set_tuning(chunk, 0)
    hl_ctx.kv_append_batch(kv, 0, shape, torch.from_numpy(kn).cuda(), torch.from_numpy(vn).cuda(), tctx, ttab)
    out = hl_ctx.attn_decode(kv, 0, shape, torch.from_numpy(qn).cuda(), tctx, int(ctxs.max()), ttab)
    got = out.cpu().numpy()
    hl_ctx.set_tuning(0, 0)
    assert_parity(got, want, "decode vs fp32 oracle")
    assert_parity(got, want16, "decode vs fp16-KV oracle", 1e-3, 6e-4)
    # the host-buffer form of the same step (append + decode, host in / host out): pageable buffers go through
    # staged copies, page-locked ones are read and written by the kernels in place; both equal the device form
    hl_ctx.set_tuning(chunk, 0)
    for pin in (False, True):
        bufs = [torch.from_numpy(x.copy()) for x in (qn, kn, vn)]
        out_h = torch.full((B, n_head, hd), float("nan"))
        if pin:
            bufs, out_h = [b.pin_memory() for b in bufs], out_h.pin_memory()
        hl_ctx.decode_step_host(kv, 0, shape, *bufs, tctx, int(ctxs.max()), ttab, out_h)
        assert np.array_equal(out_h.numpy(), got), f"host form (pinned={pin}) differs from the device form"
    hl_ctx.set_tuning(0, 0)
    kv.destroy()


def test_decode_head_dim_256_sizes_its_own_partials_scratch():
    """A context of its own, so that the split-KV partials scratch grows from nothing at head_dim 256 (it is sized in
    128-float slots: sized for 128 it made the chunks of neighbouring heads overwrite each other)."""
    ctx = hl.Context(0, torch.cuda.current_stream())
    try:
        hd, n_head, n_head_kv, bt, c = 256, 8, 2, 16, 700
        g = np.random.Generator(np.random.PCG64(256))
        theta = hl.theta_table(hd, 1e4)
        ctx.set_rope(theta)
        shape = hl.AttnShape(n_head, n_head_kv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
        nb = (c + bt - 1) // bt
        kv = ctx.kv_create(1, n_head_kv, hd, bt, nb)
        table = torch.arange(nb, dtype=torch.int32, device="cuda")
        k = g.standard_normal((c, n_head_kv, hd), dtype=np.float32)
        v = g.standard_normal((c, n_head_kv, hd), dtype=np.float32)
        q = g.standard_normal((1, n_head, hd), dtype=np.float32)
        ctx.kv_append_seq(kv, 0, shape, torch.from_numpy(k[:-1]).cuda(), torch.from_numpy(v[:-1]).cuda(), 0, table)
        tctx = torch.tensor([c], dtype=torch.int32, device="cuda")
        ctx.set_tuning(64, 0)                                  # eleven chunks per (sequence, KV head)
        ctx.kv_append_batch(kv, 0, shape, torch.from_numpy(k[-1:]).cuda(), torch.from_numpy(v[-1:]).cuda(), tctx, table.view(1, -1))
        out = ctx.attn_decode(kv, 0, shape, torch.from_numpy(q).cuda(), tctx, c, table.view(1, -1))
        want = oracle_seq(q, k[-1:], v[-1:], theta=theta, rope_mode=hl.HL_ROPE_SPLIT_HALF, prefix=(k[:-1], v[:-1]))
        assert_parity(out.cpu().numpy(), want, "head_dim 256 decode, fresh scratch")
        assert ctx.device_status() == (0, 0)
        kv.destroy()
    finally:
        ctx.close()


def test_kv_pool_with_a_kv_head_count_per_layer(hl_ctx):
    """initGpuKvCache's layerNHeadKv (naive.nim:3552-3567): three layers holding 2, 4 and (entry 0 -> the default) 2 KV
    heads.  Each layer takes the shape with ITS count -- prefill, one decode step, both against the oracle -- and
    refuses the others'; the layer sizes reported for the GpuTensor handles follow the counts."""
    hd, n_head, bt, S = 128, 8, 16, 200
    counts, given = [2, 4, 2], [2, 4, 0]
    g = np.random.Generator(np.random.PCG64(77))
    theta = hl.theta_table(hd, 1e4)
    hl_ctx.set_rope(theta)
    nb = (S + 1 + bt - 1) // bt
    kv = hl_ctx.kv_create(3, 2, hd, bt, nb, layer_n_head_kv=given)
    table = torch.from_numpy(g.permutation(nb).astype(np.int32)).cuda()
    for layer, kvh in enumerate(counts):
        assert kv.layer_ptrs(layer)[2] == nb * kvh * bt * hd * 2
        shape = hl.AttnShape(n_head, kvh, hd, hd, hl.HL_ROPE_SPLIT_HALF)
        q = g.standard_normal((S + 1, n_head, hd), dtype=np.float32)
        k = g.standard_normal((S + 1, kvh, hd), dtype=np.float32)
        v = g.standard_normal((S + 1, kvh, hd), dtype=np.float32)
        tq, tk, tv = (torch.from_numpy(x).cuda() for x in (q, k, v))
        hl_ctx.kv_append_seq(kv, layer, shape, tk[:S], tv[:S], 0, table)
        for kernel in (1, 2):
            hl_ctx.set_tuning(0, kernel)
            try:
                out = hl_ctx.attn_prefill(kv, layer, shape, tq[:S], 0, table)
            finally:
                hl_ctx.set_tuning(0, 0)
            assert_parity(out.cpu().numpy(), oracle_seq(q[:S], k[:S], v[:S], theta=theta, rope_mode=hl.HL_ROPE_SPLIT_HALF),
                          f"layer {layer} ({kvh} KV heads) prefill, kernel {kernel}")
        ctx_lens = torch.tensor([S + 1], dtype=torch.int32, device="cuda")
        hl_ctx.kv_append_batch(kv, layer, shape, tk[S:], tv[S:], ctx_lens, table.view(1, -1))
        dec = hl_ctx.attn_decode(kv, layer, shape, tq[S:], ctx_lens, S + 1, table.view(1, -1))
        assert_parity(dec.cpu().numpy(), oracle_seq(q[S:], k[S:], v[S:], theta=theta, rope_mode=hl.HL_ROPE_SPLIT_HALF,
                                                    prefix=(k[:S], v[:S])), f"layer {layer} decode")
        wrong = hl.AttnShape(n_head, 4 if kvh == 2 else 2, hd, hd, hl.HL_ROPE_SPLIT_HALF)
        with pytest.raises(hl.HlError):
            hl_ctx.attn_prefill(kv, layer, wrong, tq[:S], 0, table)
    kv.destroy()


def test_host_step_in_concurrent_slices_equals_the_device_form(hl_ctx):
    """hl_b200_decode_step_host with page-locked buffers and 40 sequences runs the batch as four concurrent chains
    (append -> decode -> combine per slice, each on its own stream, the partials scratch shared by offset): bit for bit
    the rows of the one-launch device form, two steps in a row."""
    hd, n_head, n_head_kv, bt, B = 128, 16, 4, 16, 40
    g = np.random.Generator(np.random.PCG64(4040))
    theta = hl.theta_table(hd, 5e5)
    hl_ctx.set_rope(theta)
    shape = hl.AttnShape(n_head, n_head_kv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    ctxs = g.integers(1, 900, B).astype(np.int32)
    need = (ctxs + 2 + bt - 1) // bt
    num_blocks = int(need.sum()) + 3
    perm = g.permutation(num_blocks).astype(np.int32)
    tables = np.full((B, int(need.max())), -1, np.int32)
    o = 0
    for i, n in enumerate(need):
        tables[i, :n] = perm[o:o + n]
        o += int(n)
    ttab = torch.from_numpy(tables).cuda()
    pools = [hl_ctx.kv_create(1, n_head_kv, hd, bt, num_blocks) for _ in range(2)]  # device form / host form
    prev = [(g.standard_normal((c - 1, n_head_kv, hd), dtype=np.float32), g.standard_normal((c - 1, n_head_kv, hd), dtype=np.float32))
            for c in ctxs]
    for kv in pools:
        for i, c in enumerate(ctxs):
            if c > 1:
                hl_ctx.kv_append_seq(kv, 0, shape, torch.from_numpy(prev[i][0]).cuda(), torch.from_numpy(prev[i][1]).cuda(), 0,
                                     ttab[i, :need[i]].contiguous())
    try:
        for step in range(2):
            lens = torch.from_numpy(ctxs + step).cuda()
            q = g.standard_normal((B, n_head, hd), dtype=np.float32)
            k = g.standard_normal((B, n_head_kv, hd), dtype=np.float32)
            v = g.standard_normal((B, n_head_kv, hd), dtype=np.float32)
            max_ctx = int(ctxs.max()) + step
            hl_ctx.kv_append_batch(pools[0], 0, shape, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), lens, ttab)
            dev = hl_ctx.attn_decode(pools[0], 0, shape, torch.from_numpy(q).cuda(), lens, max_ctx, ttab).cpu().numpy()
            bufs = [torch.from_numpy(x).pin_memory() for x in (q, k, v)]
            out_h = torch.full((B, n_head, hd), float("nan")).pin_memory()
            hl_ctx.decode_step_host(pools[1], 0, shape, *bufs, lens, max_ctx, ttab, out_h)
            assert np.array_equal(out_h.numpy(), dev), f"step {step}: host step in slices differs from the device form"
            if step == 0:   # and the oracle, for the longest and the shortest sequence
                for i in (int(np.argmax(ctxs)), int(np.argmin(ctxs))):
                    want = oracle_seq(q[i:i + 1], k[i:i + 1], v[i:i + 1], theta=theta, rope_mode=hl.HL_ROPE_SPLIT_HALF,
                                      prefix=prev[i] if ctxs[i] > 1 else None)[0]
                    assert_parity(out_h.numpy()[i], want, f"sequence {i} (ctx {ctxs[i]})")
    finally:
        for kv in pools:
            kv.destroy()
