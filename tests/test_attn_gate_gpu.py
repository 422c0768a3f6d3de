"""The sigmoid output gate of the qwen3.5-MoE attention layers (gpuAttnGate, naive.nim:2287-2300), fused
into the attention epilogues.  Q and gate are read straight out of a fused `[2*qDim, S]` projection buffer
laid out like the reference's (rows h*2*hd + d = Q, h*2*hd + hd + d = gate, token fastest;
naive.nim:2427-2445) through strided views -- no de-interleave copy."""
import numpy as np
import pytest
import torch

import hippo_leap_b200 as hl
import oracle
from tests.helpers import assert_parity, oracle_seq

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("S", [300, 900])   # 900: the tcgen05 kernel's tiles are two heads of one KV head there
@pytest.mark.parametrize("kernel", [1, 2], ids=["mma", "tcgen05"])
def test_prefill_gate_from_fused_q_gate_buffer(hl_ctx, kernel, S):
    H, Hkv, hd, bt = 8, 2, 128, 16
    g = np.random.Generator(np.random.PCG64(21))
    fused = g.standard_normal((H * 2 * hd, S), dtype=np.float32)     # reference layout [2*qDim, S]
    k = g.standard_normal((S, Hkv, hd), dtype=np.float32)
    v = g.standard_normal((S, Hkv, hd), dtype=np.float32)
    theta = hl.theta_table(hd, 1e6)
    hl_ctx.set_rope(theta)
    shape = hl.AttnShape(H, Hkv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    tf = torch.from_numpy(fused).cuda()
    f4 = tf.view(H, 2, hd, S)
    q_view = f4[:, 0].permute(2, 0, 1)      # [S, H, hd] view: strides (1, 2*hd*S, S)
    gate_view = f4[:, 1].permute(2, 0, 1)
    nb = (S + bt - 1) // bt
    tt = torch.randperm(nb, device="cuda").to(torch.int32)
    kv = hl_ctx.kv_create(1, Hkv, hd, bt, nb)
    hl_ctx.kv_append_seq(kv, 0, shape, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), 0, tt)
    hl_ctx.set_tuning(0, kernel)
    out = hl_ctx.attn_prefill(kv, 0, shape, q_view, 0, tt, gate=gate_view).cpu().numpy()
    hl_ctx.set_tuning(0, 0)
    f4n = fused.reshape(H, 2, hd, S)
    q = np.ascontiguousarray(f4n[:, 0].transpose(2, 0, 1))
    gate = np.ascontiguousarray(f4n[:, 1].transpose(2, 0, 1))
    want = oracle.attn_gate(oracle_seq(q, k, v, theta=theta, rope_mode=1), gate)
    assert_parity(out, want, "gated prefill")
    kv.destroy()


def test_decode_gate_single_and_multi_chunk(hl_ctx):
    H, Hkv, hd, bt = 16, 4, 64, 16
    ctxs = np.array([40, 900], np.int32)   # one single-chunk sequence (written by the decode kernel), one split
    g = np.random.Generator(np.random.PCG64(22))
    theta = hl.theta_table(hd, 1e4)
    hl_ctx.set_rope(theta)
    shape = hl.AttnShape(H, Hkv, hd, hd, hl.HL_ROPE_SPLIT_HALF)
    need = (ctxs + bt - 1) // bt
    kv = hl_ctx.kv_create(1, Hkv, hd, bt, int(need.sum()))
    tables = np.full((2, int(need.max())), -1, np.int32)
    tables[0, :need[0]] = np.arange(need[0])
    tables[1, :need[1]] = need[0] + np.arange(need[1])
    ttab = torch.from_numpy(tables).cuda()
    ks = [g.standard_normal((int(c), Hkv, hd), dtype=np.float32) for c in ctxs]
    vs = [g.standard_normal((int(c), Hkv, hd), dtype=np.float32) for c in ctxs]
    for i, c in enumerate(ctxs):
        hl_ctx.kv_append_seq(kv, 0, shape, torch.from_numpy(ks[i]).cuda(), torch.from_numpy(vs[i]).cuda(), 0,
                             ttab[i, :need[i]].contiguous())
    q = g.standard_normal((2, H, hd), dtype=np.float32)
    gate = g.standard_normal((2, H, hd), dtype=np.float32) * 2
    hl_ctx.set_tuning(64, 0)
    out = hl_ctx.attn_decode(kv, 0, shape, torch.from_numpy(q).cuda(), torch.from_numpy(ctxs).cuda(), int(ctxs.max()),
                             ttab, gate=torch.from_numpy(gate).cuda()).cpu().numpy()
    hl_ctx.set_tuning(0, 0)
    for i in range(2):
        base = oracle_seq(q[i:i + 1], ks[i][-1:], vs[i][-1:], theta=theta, rope_mode=1, prefix=(ks[i][:-1], vs[i][:-1]))
        assert_parity(out[i:i + 1], oracle.attn_gate(base, gate[i:i + 1]), f"gated decode seq {i}")
    kv.destroy()
