"""Committed golden vectors (tests/golden/attn_golden.npz, made by tests/golden/make_golden.py):
the oracle must reproduce them bit for bit on the CPU, and the CUDA path must match them within the
path's tolerance on the GPU."""
import os

import numpy as np
import pytest

import oracle
from tests.helpers import assert_parity

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_golden.npz"))
NAMES = sorted({k.split("/")[0] for k in GOLD.files})


def _case(name):
    S, H, Hkv, hd, mode, norm, steps = (int(x) for x in GOLD[f"{name}/meta"])
    qw = GOLD[f"{name}/qw"] if norm else None
    kw = GOLD[f"{name}/kw"] if norm else None
    return S, H, Hkv, hd, mode, qw, kw, steps


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("fp16", [False, True], ids=["f32", "kv16"])
def test_oracle_reproduces_golden_bit_for_bit(name, fp16):
    S, H, Hkv, hd, mode, qw, kw, steps = _case(name)
    q, k, v, theta = (GOLD[f"{name}/{x}"] for x in ("q", "k", "v", "theta"))
    assert np.array_equal(theta, oracle.theta_table(hd, _base(name)))
    cache = oracle.SeqCache(S + steps, Hkv, hd)
    outs = [oracle.attn_forward(q[:S], k[:S], v[:S], cache, theta=theta, rope_mode=mode, q_norm_w=qw, k_norm_w=kw,
                                eps=1e-6, kv_fp16=fp16)]
    for t in range(S, S + steps):
        outs.append(oracle.attn_forward(q[t:t + 1], k[t:t + 1], v[t:t + 1], cache, theta=theta, rope_mode=mode,
                                        q_norm_w=qw, k_norm_w=kw, eps=1e-6, kv_fp16=fp16))
    got = np.concatenate(outs)
    assert np.array_equal(got, GOLD[f"{name}/out_{'kv16' if fp16 else 'f32'}"])
    if not fp16:
        assert np.array_equal(cache.k, GOLD[f"{name}/k_cache"])


def _base(name):
    return {"tiny_interleaved": 1e4, "tiny_split_half": 1e4, "hd128_norm": 1e6, "single_token": 5e5}[name]


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("kernel", [1, 2, 3], ids=["mma", "tcgen05", "tcgen05-pair"])
def test_cuda_path_matches_golden(hl_ctx, name, kernel):
    import torch

    import hippo_leap_b200 as hl
    S, H, Hkv, hd, mode, qw, kw, steps = _case(name)
    if kernel == 3 and hd != 128:
        pytest.skip("the SM-pair kernel is built for head_dim 128")
    q, k, v, theta = (GOLD[f"{name}/{x}"] for x in ("q", "k", "v", "theta"))
    hl_ctx.set_rope(theta)
    shape = hl.AttnShape(H, Hkv, hd, hd, mode, 1e-6, None if qw is None else torch.from_numpy(qw).cuda(),
                         None if kw is None else torch.from_numpy(kw).cuda())
    bt = 16
    nb = (S + steps + bt - 1) // bt
    table = torch.arange(nb, dtype=torch.int32, device="cuda").flip(0).contiguous()
    kv = hl_ctx.kv_create(1, Hkv, hd, bt, nb)
    tq, tk, tv = (torch.from_numpy(x).cuda() for x in (q, k, v))
    hl_ctx.set_tuning(0, kernel)
    hl_ctx.kv_append_seq(kv, 0, shape, tk[:S], tv[:S], 0, table)
    outs = [hl_ctx.attn_prefill(kv, 0, shape, tq[:S], 0, table).cpu().numpy()]
    hl_ctx.set_tuning(0, 0)
    for t in range(S, S + steps):
        ctx_lens = torch.tensor([t + 1], dtype=torch.int32, device="cuda")
        hl_ctx.kv_append_batch(kv, 0, shape, tk[t:t + 1], tv[t:t + 1], ctx_lens, table.view(1, -1))
        outs.append(hl_ctx.attn_decode(kv, 0, shape, tq[t:t + 1], ctx_lens, t + 1, table.view(1, -1)).cpu().numpy())
    got = np.concatenate(outs)
    assert_parity(got, GOLD[f"{name}/out_f32"], f"{name} vs golden (fp32 oracle)")
    assert_parity(got, GOLD[f"{name}/out_kv16"], f"{name} vs golden (fp16-KV oracle)", 1e-3, 6e-4)
    kv.destroy()
