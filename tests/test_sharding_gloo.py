"""World-size-2 checks of the multi-GPU host logic on CPU (gloo): head sharding + one all-gather
reproduces the unsharded result; sequence sharding covers every sequence once; max-over-ranks timing."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from hippo_leap_b200 import sharding

        S, H, Hkv, hd = 24, 8, 4, 64
        g = np.random.Generator(np.random.PCG64(5))
        qa = g.standard_normal((S, H, hd), dtype=np.float32)
        ka = g.standard_normal((S, Hkv, hd), dtype=np.float32)
        va = g.standard_normal((S, Hkv, hd), dtype=np.float32)
        theta = oracle.theta_table(hd, 5e5)
        sh = sharding.head_shard(rank, world, H, Hkv)
        # each rank computes ITS heads only, from ITS slice of Q/K/V, with its own slice of the cache
        cache = oracle.SeqCache(S, sh.n_head_kv, hd)
        out_l = oracle.attn_forward(qa[:, sh.q_lo:sh.q_hi], ka[:, sh.kv_lo:sh.kv_hi], va[:, sh.kv_lo:sh.kv_hi], cache,
                                    theta=theta, rope_mode=1, n_threads=1)
        head_major = torch.from_numpy(np.ascontiguousarray(out_l.transpose(1, 0, 2)))  # [H/N, S, hd]
        full = sharding.gather_heads(head_major)
        want = oracle.attn_forward(qa, ka, va, oracle.SeqCache(S, Hkv, hd), theta=theta, rope_mode=1, n_threads=1)
        ok_gather = bool(np.array_equal(full.numpy(), want.transpose(1, 0, 2)))
        # one batched decode step, head-sharded: every rank holds its KV heads of EVERY sequence, attends with its query
        # heads, and one all-gather of the head-major rows gives the unsharded step
        ctxs = [5, 17, 9]
        qd = g.standard_normal((len(ctxs), 1, H, hd), dtype=np.float32)
        loc, ref = [], []
        for i, c in enumerate(ctxs):
            kk = g.standard_normal((c, Hkv, hd), dtype=np.float32)
            vv = g.standard_normal((c, Hkv, hd), dtype=np.float32)
            for lo_q, hi_q, lo_kv, hi_kv, dst in ((sh.q_lo, sh.q_hi, sh.kv_lo, sh.kv_hi, loc), (0, H, 0, Hkv, ref)):
                sc = oracle.SeqCache(c, hi_kv - lo_kv, hd)
                if c > 1:
                    oracle.attn_forward(np.zeros((c - 1, hi_q - lo_q, hd), np.float32), kk[:-1, lo_kv:hi_kv],
                                        vv[:-1, lo_kv:hi_kv], sc, theta=theta, rope_mode=1, rows=[[0, 0]], n_threads=1)
                dst.append(oracle.attn_forward(qd[i][:, lo_q:hi_q], kk[-1:, lo_kv:hi_kv], vv[-1:, lo_kv:hi_kv], sc,
                                               theta=theta, rope_mode=1, n_threads=1)[0])
        dec_local = torch.from_numpy(np.ascontiguousarray(np.stack(loc).transpose(1, 0, 2)))  # [H/N, B, hd]
        ok_gather = ok_gather and bool(np.array_equal(sharding.gather_heads(dec_local).numpy(),
                                                      np.stack(ref).transpose(1, 0, 2)))
        # sequence sharding: identical on every rank, disjoint, complete
        ctx = g.integers(512, 8193, 64)
        owners = sharding.shard_sequences(ctx, world)
        flat = sorted(i for o in owners for i in o)
        loads = [int(ctx[o].sum()) for o in owners]
        ok_seq = flat == list(range(64)) and max(loads) - min(loads) <= int(ctx.max())
        slow = sharding.max_over_ranks(1.0 + rank, torch.device("cpu"))
        q.put((rank, ok_gather, ok_seq, slow))
    finally:
        dist.destroy_process_group()


def test_head_sharding_allgather_and_sequence_sharding_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_gather, ok_seq, slow in res:
        assert ok_gather, f"rank {rank}: gathered heads differ from the unsharded oracle"
        assert ok_seq, f"rank {rank}: sequence sharding broken"
        assert slow == 2.0


def test_head_shard_arithmetic_and_errors():
    sys.path.insert(0, ROOT)
    from hippo_leap_b200 import sharding
    for world in (1, 2, 4, 8):
        seen_q, seen_kv = [], []
        for r in range(world):
            sh = sharding.head_shard(r, world, 64, 8)
            seen_q += list(range(sh.q_lo, sh.q_hi))
            seen_kv += list(range(sh.kv_lo, sh.kv_hi))
            for hq in range(sh.q_lo, sh.q_hi):  # a query head's KV head lives on the same rank
                assert sh.kv_lo <= hq // 8 < sh.kv_hi
        assert seen_q == list(range(64)) and seen_kv == list(range(8))
    with pytest.raises(ValueError):
        sharding.head_shard(0, 3, 64, 8)
    with pytest.raises(ValueError):
        sharding.head_shard(0, 2, 6, 4)


def test_sharded_decode_workload_is_one_seeded_set_balanced_by_bytes():
    sys.path.insert(0, ROOT)
    from hippo_leap_b200 import synth
    cfg = synth.CONFIGS[4]
    one, owners1 = synth.gen_sharded_ctx_lens(cfg, 1)
    assert np.array_equal(one, synth.gen_ctx_lens(cfg)) and owners1 == [list(range(cfg.batch))]
    for world in (2, 4, 8):
        all_ctx, owners = synth.gen_sharded_ctx_lens(cfg, world)
        assert np.array_equal(all_ctx[:cfg.batch], one)          # the one-GPU set is a prefix of every larger set
        assert sorted(i for o in owners for i in o) == list(range(cfg.batch * world))
        for o in owners:                                         # weak scaling: every rank carries the one-GPU work
            assert len(o) == cfg.batch and np.array_equal(np.sort(all_ctx[o]), np.sort(one))
    # the dealing rule itself on an uneven set: KV bytes per rank within 1 % of the mean
    g = np.random.Generator(np.random.PCG64(9))
    ctx = g.integers(512, 8193, 512)
    loads = np.array([int(ctx[o].sum()) for o in synth.shard_longest_first(ctx, 8)])
    assert loads.max() / loads.mean() < 1.01
