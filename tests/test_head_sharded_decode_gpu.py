"""KV-head-sharded batched decode on one GPU: the shards of a world of 1, 2, 4 and 8 ranks are run one after the
other (each on a pool that holds only its KV heads of every sequence's pages), their head-major rows are
concatenated in rank order -- what the single all-gather does -- and the result is compared with the oracle and,
bit for bit, with the unsharded decode step.  The variant whose kernels store to extra destinations must put
identical rows into each of them."""
import numpy as np
import pytest
import torch

import hippo_leap_b200 as hl
from hippo_leap_b200 import sharding
from tests.helpers import assert_parity, oracle_seq

pytestmark = pytest.mark.gpu


def _workload(seed, n_head, n_head_kv, hd, ctxs, bt):
    g = np.random.Generator(np.random.PCG64(seed))
    ctxs = np.asarray(ctxs, np.int32)
    need = (ctxs + bt - 1) // bt
    num_blocks = int(need.sum()) + 2
    perm = g.permutation(num_blocks).astype(np.int32)
    tables = np.full((len(ctxs), int(need.max())), -1, np.int32)
    o = 0
    for i, n in enumerate(need):
        tables[i, :n] = perm[o:o + n]
        o += int(n)
    ks = [g.standard_normal((int(c), n_head_kv, hd), dtype=np.float32) for c in ctxs]
    vs = [g.standard_normal((int(c), n_head_kv, hd), dtype=np.float32) for c in ctxs]
    q = g.standard_normal((len(ctxs), n_head, hd), dtype=np.float32)
    return ctxs, need, num_blocks, tables, ks, vs, q


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_head_sharded_decode_equals_unsharded_and_oracle(hl_ctx, world):
    n_head, n_head_kv, hd, bt = 32, 8, 128, 16
    ctxs, need, num_blocks, tables, ks, vs, q = _workload([world, 7], n_head, n_head_kv, hd,
                                                          [700, 64, 1, 2049, 333, 1500, 17], bt)
    B = len(ctxs)
    theta = hl.theta_table(hd, 5e5)
    hl_ctx.set_rope(theta)
    ttab, tctx = torch.from_numpy(tables).cuda(), torch.from_numpy(ctxs).cuda()
    max_ctx = int(ctxs.max())
    hl_ctx.set_tuning(256, 0)   # the same chunks whatever the number of local KV heads: bit-equal summation order
    try:
        def run_shard(sh):
            """Fill a pool with this shard's KV heads (all but the newest token), then one sharded decode step."""
            shape = hl.AttnShape(sh.n_head, sh.n_head_kv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
            kv = hl_ctx.kv_create(1, sh.n_head_kv, hd, bt, num_blocks)
            for i, c in enumerate(ctxs):
                if c > 1:
                    hl_ctx.kv_append_seq(kv, 0, shape, torch.from_numpy(ks[i][:-1, sh.kv_lo:sh.kv_hi]).cuda(),
                                         torch.from_numpy(vs[i][:-1, sh.kv_lo:sh.kv_hi]).cuda(), 0,
                                         ttab[i, :need[i]].contiguous())
            runner = sharding.HeadShardedDecode(hl_ctx, kv, shape, B, torch.device("cuda"), world=1)
            k_new = torch.from_numpy(np.stack([k[-1, sh.kv_lo:sh.kv_hi] for k in ks])).cuda()
            v_new = torch.from_numpy(np.stack([v[-1, sh.kv_lo:sh.kv_hi] for v in vs])).cuda()
            rows = runner.run(torch.from_numpy(q[:, sh.q_lo:sh.q_hi]).cuda(), k_new, v_new, tctx, max_ctx, ttab).clone()
            # the broadcasting variant: same rows in `out` and in two more destinations
            bufs = [torch.zeros_like(rows) for _ in range(3)]
            hl_ctx.attn_decode_bcast(kv, 0, shape, torch.from_numpy(q[:, sh.q_lo:sh.q_hi]).cuda(), tctx, max_ctx, ttab,
                                     bufs[0].permute(1, 0, 2), [b.data_ptr() for b in bufs[1:]])
            torch.cuda.synchronize()
            for b in bufs:
                assert torch.equal(b, rows)
            kv.destroy()
            return rows                                                   # [n_head / world, B, hd]

        gathered = torch.cat([run_shard(sharding.head_shard(r, world, n_head, n_head_kv)) for r in range(world)])
        whole = run_shard(sharding.head_shard(0, 1, n_head, n_head_kv))
    finally:
        hl_ctx.set_tuning(0, 0)
    assert gathered.shape == (n_head, B, hd)
    assert torch.equal(gathered, whole), "rank-order concatenation of the shards differs from the unsharded step"
    got = gathered.permute(1, 0, 2).cpu().numpy()
    for i, c in enumerate(ctxs):
        want = oracle_seq(q[i:i + 1], ks[i][-1:], vs[i][-1:], theta=theta, rope_mode=1,
                          prefix=(ks[i][:-1], vs[i][:-1]) if c > 1 else None)
        assert_parity(got[i:i + 1], want, f"head-sharded decode, world {world}, sequence {i} (ctx {c})")


def test_decode_bcast_refuses_bad_peer_lists(hl_ctx):
    n_head, n_head_kv, hd, bt = 8, 2, 64, 16
    hl_ctx.set_rope(hl.theta_table(hd, 1e4))
    shape = hl.AttnShape(n_head, n_head_kv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    kv = hl_ctx.kv_create(1, n_head_kv, hd, bt, 4)
    ttab = torch.zeros((1, 4), dtype=torch.int32, device="cuda")
    tctx = torch.full((1,), 20, dtype=torch.int32, device="cuda")
    q = torch.zeros((1, n_head, hd), device="cuda")
    out = torch.zeros_like(q)
    launches = hl_ctx.launch_count()
    try:
        with pytest.raises(hl.HlError) as ei:
            hl_ctx.attn_decode_bcast(kv, 0, shape, q, tctx, 20, ttab, out, [out.data_ptr()] * 8)
        assert ei.value.code == 1   # HL_ERR_ARG: more than 7 peers
        with pytest.raises(hl.HlError) as ei:
            hl_ctx.attn_decode_bcast(kv, 0, shape, q, tctx, 20, ttab, out, [out.data_ptr() + 2])
        assert ei.value.code == 3   # HL_ERR_ALIGN
        assert hl_ctx.launch_count() == launches
    finally:
        kv.destroy()
