"""Failure detection without faulting a GPU.

CPU: every entry point refuses bad arguments with a status code before it touches a device.
GPU: host-side argument checks on a live context; a bounded device-side wait that runs out reports
HL_ERR_TIMEOUT through the status word; a bad block-table entry reports HL_ERR_BOUNDS and is clamped.
In every case the context stays usable afterwards (a small decode step still matches the oracle)."""
import ctypes as C

import numpy as np
import pytest

from hippo_leap_b200 import _lib as L


def test_null_context_is_refused_everywhere_without_a_gpu():
    lib = L.load()
    null = C.c_void_p(None)
    assert lib.hl_b200_destroy(null) == L.HL_ERR_ARG
    assert lib.hl_b200_sync(null) == L.HL_ERR_ARG
    assert lib.hl_b200_set_stream(null, null) == L.HL_ERR_ARG
    assert lib.hl_b200_set_rope(null, None, 4) == L.HL_ERR_ARG
    assert lib.hl_b200_set_tuning(null, 0, 0) == L.HL_ERR_ARG
    assert lib.hl_b200_selftest_wait_timeout(null, 10) == L.HL_ERR_ARG
    out = C.c_void_p()
    assert lib.hl_b200_kv_create(null, 1, 1, 64, 16, 1, C.byref(out)) == L.HL_ERR_ARG
    assert lib.hl_b200_kv_destroy(null, null) == L.HL_ERR_ARG
    assert lib.hl_b200_kv_layer(null, 0, None, None, None) == L.HL_ERR_ARG
    assert lib.hl_b200_attn_decode(null, null, 0, None, None, 1, null, 1, null, 1, None, None) == L.HL_ERR_ARG
    assert lib.hl_b200_attn_decode_static(null, null, 0, None, None, 1, null, 1, null, 1, None) == L.HL_ERR_ARG
    assert lib.hl_b200_attn_prefill(null, null, 0, None, None, 1, 0, null, 1, None, None) == L.HL_ERR_ARG
    assert lib.hl_b200_kv_append_seq(null, null, 0, None, None, None, 1, 0, null, 1) == L.HL_ERR_ARG
    assert lib.hl_b200_kv_append_batch(null, null, 0, None, None, None, 1, null, null, 1) == L.HL_ERR_ARG
    assert lib.hl_b200_prefill_host(null, null, 0, None, None, None, None, 1, 0, null, 1, None, None) == L.HL_ERR_ARG
    assert lib.hl_b200_decode_step_host(null, null, 0, None, None, None, None, 1, null, 1, null, 1, None, None) == L.HL_ERR_ARG
    assert lib.hl_b200_launch_count(null) == -1
    assert lib.hl_b200_last_error(null) == b"null context"
    th = (C.c_float * 4)()
    assert lib.hl_b200_theta_table_h(1e4, 7, th) == L.HL_ERR_ARG      # odd rope_dim
    assert lib.hl_b200_theta_table_h(-1.0, 8, th) == L.HL_ERR_ARG     # non-positive base
    assert lib.hl_b200_theta_llama3_scale_h(th, 4, 32.0, 4.0, 1.0, 8192) == L.HL_ERR_ARG  # high <= low


def _small_case(hl_ctx, bad_entry=None):
    import torch

    import hippo_leap_b200 as hl
    hd, H, Hkv, bt, ctxs = 64, 8, 2, 16, np.array([40, 17], np.int32)
    g = np.random.Generator(np.random.PCG64(3))
    theta = hl.theta_table(hd, 1e4)
    hl_ctx.set_rope(theta)
    shape = hl.AttnShape(H, Hkv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    kv = hl_ctx.kv_create(1, Hkv, hd, bt, 8)
    tables = np.array([[0, 1, 2], [3, 4, -1]], np.int32)
    k = [g.standard_normal((int(c), Hkv, hd), dtype=np.float32) for c in ctxs]
    v = [g.standard_normal((int(c), Hkv, hd), dtype=np.float32) for c in ctxs]
    q = g.standard_normal((2, H, hd), dtype=np.float32)
    ttab = torch.from_numpy(tables).cuda()
    for i, c in enumerate(ctxs):
        hl_ctx.kv_append_seq(kv, 0, shape, torch.from_numpy(k[i]).cuda(), torch.from_numpy(v[i]).cuda(), 0,
                             ttab[i, :(int(c) + bt - 1) // bt].contiguous())
    if bad_entry is not None:
        tables = tables.copy()
        tables[0, 1] = bad_entry
        ttab = torch.from_numpy(tables).cuda()
    return hl, torch, shape, kv, ttab, torch.from_numpy(ctxs).cuda(), ctxs, q, k, v, theta


def _decode_matches_oracle(hl_ctx):
    from tests.helpers import assert_parity, oracle_seq
    hl, torch, shape, kv, ttab, tctx, ctxs, q, k, v, theta = _small_case(hl_ctx)
    out = hl_ctx.attn_decode(kv, 0, shape, torch.from_numpy(q).cuda(), tctx, int(ctxs.max()), ttab).cpu().numpy()
    for i in range(2):
        want = oracle_seq(q[i:i + 1], k[i][-1:], v[i][-1:], theta=theta, rope_mode=1, prefix=(k[i][:-1], v[i][:-1]))
        assert_parity(out[i:i + 1], want, "decode after a failure path")
    kv.destroy()


@pytest.mark.gpu
def test_bounded_wait_times_out_with_status_and_context_survives(hl_ctx, request):
    request.node.add_marker("expects_device_status")
    hl_ctx.selftest_wait_timeout(2000)
    code, detail = hl_ctx.device_status()
    assert (code, detail) == (L.HL_ERR_TIMEOUT, 900)
    assert hl_ctx.device_status() == (0, 0)  # reading clears it
    _decode_matches_oracle(hl_ctx)


@pytest.mark.gpu
@pytest.mark.parametrize("bad", [-1, 8, 10 ** 6])
def test_bad_block_table_entry_reports_bounds_and_does_not_fault(hl_ctx, bad):
    import hippo_leap_b200 as hl
    hl_mod, torch, shape, kv, ttab, tctx, ctxs, q, k, v, theta = _small_case(hl_ctx, bad_entry=bad)
    tq = torch.from_numpy(q).cuda()
    hl_ctx.attn_decode(kv, 0, shape, tq, tctx, int(ctxs.max()), ttab)
    assert hl_ctx.device_status()[0] == L.HL_ERR_BOUNDS
    for kernel in (1, 2):
        hl_ctx.set_tuning(0, kernel)
        hl_ctx.attn_prefill(kv, 0, shape, torch.from_numpy(np.repeat(q[:1], 40, 0)).cuda(), 0, ttab[0].contiguous())
        assert hl_ctx.device_status()[0] == L.HL_ERR_BOUNDS
    hl_ctx.set_tuning(0, 0)
    knew = torch.from_numpy(k[0][:1]).cuda()
    hl_ctx.kv_append_seq(kv, 0, shape, knew, knew, 16, ttab[0].contiguous())  # position 16 -> the bad entry
    assert hl_ctx.device_status()[0] == L.HL_ERR_BOUNDS
    kv.destroy()
    _decode_matches_oracle(hl_ctx)


@pytest.mark.gpu
def test_host_side_argument_matrix_on_a_live_context(hl_ctx):
    import torch

    import hippo_leap_b200 as hl
    hl_mod, _, shape, kv, ttab, tctx, ctxs, q, k, v, theta = _small_case(hl_ctx)
    tq = torch.from_numpy(q).cuda()
    launches = hl_ctx.launch_count()

    def refuse(code, fn):
        with pytest.raises(hl.HlError) as ei:
            fn()
        assert ei.value.code == code, ei.value

    bad_heads = hl.AttnShape(7, 2, 64, 64, hl.HL_ROPE_SPLIT_HALF)
    refuse(L.HL_ERR_ARG, lambda: hl_ctx.attn_decode(kv, 0, bad_heads, tq, tctx, 40, ttab))
    refuse(L.HL_ERR_ARG, lambda: hl_ctx.attn_decode(kv, 3, shape, tq, tctx, 40, ttab))            # layer
    refuse(L.HL_ERR_CAPACITY, lambda: hl_ctx.attn_decode(kv, 0, shape, tq, tctx, 49, ttab))       # ctx > table
    refuse(L.HL_ERR_ARG, lambda: hl_ctx.attn_decode(kv, 0, shape, tq, tctx, 0, ttab))
    other_dim = hl.AttnShape(8, 2, 128, 128, hl.HL_ROPE_SPLIT_HALF)
    refuse(L.HL_ERR_ARG, lambda: hl_ctx.attn_decode(kv, 0, other_dim, tq, tctx, 40, ttab))        # pool is hd 64
    odd_rope = hl.AttnShape(8, 2, 64, 31, hl.HL_ROPE_SPLIT_HALF)
    refuse(L.HL_ERR_ARG, lambda: hl_ctx.attn_prefill(kv, 0, odd_rope, tq, 0, ttab[0].contiguous()))
    refuse(L.HL_ERR_CAPACITY, lambda: hl_ctx.attn_prefill(kv, 0, shape, tq, 47, ttab[0].contiguous()))
    refuse(L.HL_ERR_ARG, lambda: hl_ctx.attn_prefill(kv, 0, shape, tq, -1, ttab[0].contiguous()))
    refuse(L.HL_ERR_CAPACITY, lambda: hl_ctx.kv_append_seq(kv, 0, shape, tq[:, :2], tq[:, :2], 47, ttab[0].contiguous()))
    refuse(L.HL_ERR_UNSUPPORTED, lambda: hl_ctx.kv_create(1, 2, 96, 16, 4))
    refuse(L.HL_ERR_ARG, lambda: hl_ctx.kv_create(1, 2, 64, 24, 4))                               # block_tokens % 16
    refuse(L.HL_ERR_ARG, lambda: hl_ctx.set_tuning(100, 0))
    refuse(L.HL_ERR_ARG, lambda: hl_ctx.attn_decode(kv, 0, shape, tq.to(torch.float64), tctx, 40, ttab))
    assert hl_ctx.launch_count() == launches, "a refused call must not launch anything"
    kv.destroy()


@pytest.mark.gpu
def test_device_side_context_length_beyond_the_grid_reports_bounds(hl_ctx, request):
    """ctx_lens lives on the device; the host sizes the grid and the partial slots from max_ctx_h.  A context longer
    than that (a stale host value, a caller mistake) is reported through the status word and clamped to the grid, an
    empty one is reported and its output row zeroed -- no read outside the partial slots, the context stays usable."""
    request.node.add_marker("expects_device_status")
    import torch

    import hippo_leap_b200 as hl
    hd, H, Hkv, bt = 128, 8, 2, 16
    ctxs = np.array([600, 130], np.int32)
    g = np.random.Generator(np.random.PCG64(31))
    hl_ctx.set_rope(hl.theta_table(hd, 1e4))
    shape = hl.AttnShape(H, Hkv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    nb = (int(ctxs.max()) + bt - 1) // bt
    kv = hl_ctx.kv_create(1, Hkv, hd, bt, 2 * nb)
    tables = np.arange(2 * nb, dtype=np.int32).reshape(2, nb)
    ttab, tctx = torch.from_numpy(tables).cuda(), torch.from_numpy(ctxs).cuda()
    for i, c in enumerate(ctxs):
        k = torch.from_numpy(g.standard_normal((int(c), Hkv, hd), dtype=np.float32)).cuda()
        hl_ctx.kv_append_seq(kv, 0, shape, k, k, 0, ttab[i].contiguous())
    q = torch.from_numpy(g.standard_normal((2, H, hd), dtype=np.float32)).cuda()
    hl_ctx.set_tuning(128, 0)
    try:
        good = hl_ctx.attn_decode(kv, 0, shape, q, tctx, 600, ttab).clone()
        assert hl_ctx.device_status() == (0, 0)
        # max_ctx_h understated by more than one chunk: 3 chunks of 128 on the grid, sequence 0 has 600 keys
        out = hl_ctx.attn_decode(kv, 0, shape, q, tctx, 384, ttab)
        assert hl_ctx.device_status() == (L.HL_ERR_BOUNDS, 0)
        assert torch.isfinite(out).all()
        assert torch.equal(out[1], good[1])      # the sequence that fits is untouched
        # an empty context: reported, output row zeroed
        empty = torch.tensor([0, 130], dtype=torch.int32, device="cuda")
        out = torch.full_like(good, float("nan"))
        hl_ctx.attn_decode(kv, 0, shape, q, empty, 600, ttab, out)
        assert hl_ctx.device_status() == (L.HL_ERR_BOUNDS, 0)
        assert float(out[0].abs().max()) == 0.0 and torch.equal(out[1], good[1])
        again = hl_ctx.attn_decode(kv, 0, shape, q, tctx, 600, ttab)
        assert torch.equal(again, good) and hl_ctx.device_status() == (0, 0)
    finally:
        hl_ctx.set_tuning(0, 0)
        kv.destroy()
