"""The allocation-free decode entry point (hl_b200_attn_decode_static), through the C ABI.

Some callers cannot let the library allocate: a serving process that has given all device memory to
its own KV arena, or a decode loop that must never hit cudaMalloc's device-wide synchronisation.  For
them the split-KV scratch is a fixed array inside the library.  This file checks, on two calls in a
row (the second with other queries, so stale scratch contents would show), that the result equals the
regular entry point's, and that a request beyond the fixed scratch is refused with a clear error.
It is collected last on purpose: a run that stops at the first failure has then run everything else.
"""
import numpy as np
import pytest
import torch

import hippo_leap_b200 as hl
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu


def _fill(hl_ctx, shape, kv, ttab, ctxs, bt, g):
    for i, c in enumerate(ctxs):
        k = torch.from_numpy(g.standard_normal((int(c), shape.n_head_kv, shape.head_dim), dtype=np.float32)).cuda()
        v = torch.from_numpy(g.standard_normal((int(c), shape.n_head_kv, shape.head_dim), dtype=np.float32)).cuda()
        nb = (int(c) + bt - 1) // bt
        hl_ctx.kv_append_seq(kv, 0, shape, k, v, 0, ttab[i, :nb].contiguous())


@pytest.mark.parametrize("hd,n_head,n_head_kv,ctxs,chunk", [
    (128, 32, 8, [700, 64, 1, 2049, 333, 1500], 0),
    (64, 32, 4, [129, 4000], 256),
])
def test_static_decode_matches_regular_entry_point_twice(hl_ctx, hd, n_head, n_head_kv, ctxs, chunk):
    bt = 16
    g = np.random.Generator(np.random.PCG64([hd, 9]))
    ctxs = np.asarray(ctxs, np.int32)
    hl_ctx.set_rope(hl.theta_table(hd, 5e5))
    shape = hl.AttnShape(n_head, n_head_kv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    need = (ctxs + bt - 1) // bt
    num_blocks = int(need.sum()) + 3
    perm = g.permutation(num_blocks).astype(np.int32)
    tables = np.full((len(ctxs), int(need.max())), -1, np.int32)
    o = 0
    for i, n in enumerate(need):
        tables[i, :n] = perm[o:o + n]
        o += int(n)
    ttab = torch.from_numpy(tables).cuda()
    tctx = torch.from_numpy(ctxs).cuda()
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, num_blocks)
    _fill(hl_ctx, shape, kv, ttab, ctxs, bt, g)
    hl_ctx.set_tuning(chunk, 0)
    try:
        for call in range(2):
            q = torch.from_numpy(g.standard_normal((len(ctxs), n_head, hd), dtype=np.float32)).cuda()
            want = hl_ctx.attn_decode(kv, 0, shape, q, tctx, int(ctxs.max()), ttab)
            got = torch.full_like(want, float("nan"))
            hl_ctx.attn_decode_static(kv, 0, shape, q, tctx, int(ctxs.max()), ttab, got)
            torch.cuda.synchronize()
            assert_parity(got.cpu().numpy(), want.cpu().numpy(), f"static decode, call {call}")
            # both entry points cut the context into the same chunks, so they agree bit for bit
            assert torch.equal(got, want)
        # fp16 query in, fp16 result out
        q16 = q.half()
        want16 = torch.empty_like(q16)
        hl_ctx.attn_decode(kv, 0, shape, q16, tctx, int(ctxs.max()), ttab, want16)
        got16 = torch.full_like(want16, float("nan"))
        hl_ctx.attn_decode_static(kv, 0, shape, q16, tctx, int(ctxs.max()), ttab, got16)
        torch.cuda.synchronize()
        assert torch.equal(got16, want16)
        assert_parity(got16.float().cpu().numpy(), want.cpu().numpy(), "static decode, fp16 in/out", 6e-3, 3e-3)
    finally:
        hl_ctx.set_tuning(0, 0)
        kv.destroy()


def test_static_decode_rejects_requests_beyond_the_fixed_scratch(hl_ctx):
    hd, n_head, n_head_kv, bt = 64, 64, 4, 16
    hl_ctx.set_rope(hl.theta_table(hd, 1e4))
    shape = hl.AttnShape(n_head, n_head_kv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    batch, ctx = 64, 1024           # 64-token chunks -> 16 chunks: 64 * 64 * 16 = 65536 slots > 32768
    nb = ctx // bt
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, 8)
    ttab = torch.zeros((batch, nb), dtype=torch.int32, device="cuda")
    tctx = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
    q = torch.zeros((batch, n_head, hd), device="cuda")
    out = torch.zeros_like(q)
    hl_ctx.set_tuning(64, 0)
    try:
        with pytest.raises(hl.HlError, match="static scratch holds") as ei:
            hl_ctx.attn_decode_static(kv, 0, shape, q, tctx, ctx, ttab, out)
        assert ei.value.code == 2  # HL_ERR_CAPACITY
    finally:
        hl_ctx.set_tuning(0, 0)
        kv.destroy()


def test_static_decode_refuses_bad_views_like_the_regular_entry_point(hl_ctx):
    """A view whose pointer is not aligned to its element size, or whose dtype is unknown, comes back as a status
    code before anything is launched -- the same checks as hl_b200_attn_decode."""
    import ctypes as C

    from hippo_leap_b200 import _lib as L
    from hippo_leap_b200.runtime import view_of
    hd, n_head, n_head_kv, bt = 64, 8, 2, 16
    hl_ctx.set_rope(hl.theta_table(hd, 1e4))
    shape = hl.AttnShape(n_head, n_head_kv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, 4)
    ttab = torch.zeros((1, 4), dtype=torch.int32, device="cuda")
    tctx = torch.full((1,), 20, dtype=torch.int32, device="cuda")
    q = torch.zeros((1, n_head, hd), device="cuda")
    out = torch.zeros_like(q)
    launches = hl_ctx.launch_count()
    sc = shape.c()

    def call(qv, ov):
        return hl_ctx.lib.hl_b200_attn_decode_static(hl_ctx.handle, kv.handle, 0, C.byref(sc), C.byref(qv), 1,
                                                     tctx.data_ptr(), 20, ttab.data_ptr(), 4, C.byref(ov))

    try:
        odd = view_of(q)
        odd.ptr = q.data_ptr() + 2               # a float32 view at an address that is not a multiple of 4
        assert call(odd, view_of(out)) == L.HL_ERR_ALIGN
        odd_out = view_of(out)
        odd_out.ptr = out.data_ptr() + 1
        assert call(view_of(q), odd_out) == L.HL_ERR_ALIGN
        bad_dtype = view_of(q)
        bad_dtype.dtype = 5
        assert call(bad_dtype, view_of(out)) == L.HL_ERR_ARG
        assert hl_ctx.launch_count() == launches, "a refused call must not launch anything"
        assert call(view_of(q), view_of(out)) == 0   # the same arguments, well-formed, are accepted
    finally:
        kv.destroy()
