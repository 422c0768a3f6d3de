"""CPU checks of the oracle itself: each tensor.nim primitive against numpy float64, the
attention glue against an independent float64 computation, and internal consistency."""
import numpy as np
import pytest

import oracle


def rng(seed=0):
    return np.random.Generator(np.random.PCG64(seed))


def test_matmul_matches_float64():
    g = rng(1)
    a = g.standard_normal((7, 33), dtype=np.float32)
    b = g.standard_normal((33, 5), dtype=np.float32)
    c = oracle.matmul(a, b)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(c - ref).max() < 2e-5
    # k-innermost sequential float32 accumulation, exactly as tensor.nim:77-80
    acc = np.float32(0)
    for p in range(33):
        acc = np.float32(acc + np.float32(a[2, p] * b[p, 3]))
    assert c[2, 3] == acc


def test_rmsnorm_formula():
    g = rng(2)
    x = g.standard_normal((3, 4, 128), dtype=np.float32)
    w = g.uniform(0.9, 1.1, 128).astype(np.float32)
    out = oracle.rmsnorm(x, w, 1e-6)
    x64 = x.astype(np.float64)
    ref = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-6) * w
    assert np.abs(out - ref).max() < 1e-5


def test_softmax_rows_sum_to_one_and_match():
    g = rng(3)
    x = (g.standard_normal((5, 77), dtype=np.float32) * 4).astype(np.float32)
    p = oracle.softmax_last_dim(x)
    e = np.exp(x.astype(np.float64) - x.max(-1, keepdims=True))
    assert np.abs(p - e / e.sum(-1, keepdims=True)).max() < 1e-6
    assert np.abs(p.sum(-1) - 1).max() < 1e-5
    # a single -1e30 style masked entry contributes exactly zero
    x[:, 10] = -1e30
    assert (oracle.softmax_last_dim(x)[:, 10] == 0).all()


@pytest.mark.parametrize("base,dim,start", [(1e4, 64, 0), (5e5, 128, 1000), (1e6, 128, 32000)])
def test_rope_inplace_equals_theta_table_path(base, dim, start):
    g = rng(4)
    x = g.standard_normal((2, 9, dim), dtype=np.float32)
    y = x.copy()
    oracle.rope_inplace(x, base, start)
    th = oracle.theta_table(dim, base)
    for o in range(2):
        for p in range(9):
            oracle.rope_row(y[o, p], dim, th, start + p, oracle.ROPE_INTERLEAVED)
    assert np.array_equal(x, y)  # bit-identical: same theta, same one-multiply angle, same libm
    # against float64 rotation
    z = g.standard_normal((1, 1, dim), dtype=np.float32)
    z0 = z.copy()
    oracle.rope_inplace(z, base, start)
    ang = np.float64(np.float32(start)) * th.astype(np.float64)
    a, b = z0[0, 0, 0::2].astype(np.float64), z0[0, 0, 1::2].astype(np.float64)
    # the float32 angle is rounded before sin/cos, so compare with the rounded angle
    ang32 = (np.float32(start) * th).astype(np.float64)
    assert np.abs(z[0, 0, 0::2] - (a * np.cos(ang32) - b * np.sin(ang32))).max() < 1e-5
    assert np.abs(ang - ang32).max() <= np.abs(ang).max() * 2 ** -23


def test_rope_split_half_leaves_tail_untouched():
    g = rng(5)
    x = g.standard_normal(128, dtype=np.float32)
    y = x.copy()
    th = oracle.theta_table(64, 1e4)
    oracle.rope_row(y, 64, th, 7, oracle.ROPE_SPLIT_HALF)
    assert np.array_equal(x[64:], y[64:])
    ang = (np.float32(7) * th).astype(np.float64)
    assert np.abs(y[:32] - (x[:32] * np.cos(ang) - x[32:64] * np.sin(ang))).max() < 1e-6
    assert np.abs(y[32:64] - (x[:32] * np.sin(ang) + x[32:64] * np.cos(ang))).max() < 1e-6


def _ref64(q, k, v, theta, mode, qw=None, kw=None, eps=1e-6, start=0):
    S, H, hd = q.shape
    Hkv = k.shape[1]
    half = hd // 2

    def norm(x, w):
        if w is None:
            return x.astype(np.float64)
        x = x.astype(np.float64)
        return x / np.sqrt((x ** 2).mean(-1, keepdims=True) + eps) * w

    def rope(x, pos):
        x = x.copy()
        ang = (pos.astype(np.float32)[:, None] * theta[None, :]).astype(np.float64)
        cs, sn = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        if mode == 0:
            a, b = x[..., 0::2].copy(), x[..., 1::2].copy()
            x[..., 0::2], x[..., 1::2] = a * cs - b * sn, a * sn + b * cs
        else:
            a, b = x[..., :half].copy(), x[..., half:].copy()
            x[..., :half], x[..., half:] = a * cs - b * sn, a * sn + b * cs
        return x

    pos = np.arange(start, start + S)
    qr, kr = rope(norm(q, qw), pos), rope(norm(k, kw), pos)
    out = np.zeros((S, H, hd))
    for h in range(H):
        kh = h // (H // Hkv)
        s = qr[:, h] @ kr[:, kh].T / np.sqrt(hd)
        s = np.where(np.tril(np.ones((S, S))) > 0, s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        out[:, h] = p @ v[:, kh].astype(np.float64)
    return out


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("norm", [False, True])
def test_attention_glue_against_float64(mode, norm):
    g = rng(6)
    S, H, Hkv, hd = 48, 8, 2, 64
    q = g.standard_normal((S, H, hd), dtype=np.float32)
    k = g.standard_normal((S, Hkv, hd), dtype=np.float32)
    v = g.standard_normal((S, Hkv, hd), dtype=np.float32)
    qw = g.uniform(0.9, 1.1, hd).astype(np.float32) if norm else None
    kw = g.uniform(0.9, 1.1, hd).astype(np.float32) if norm else None
    th = oracle.theta_table(hd, 1e4)
    c = oracle.SeqCache(S, Hkv, hd)
    out = oracle.attn_forward(q, k, v, c, theta=th, rope_mode=mode, q_norm_w=qw, k_norm_w=kw)
    assert np.abs(out - _ref64(q, k, v, th, mode, qw, kw)).max() < 5e-6
    assert c.cur_len == S


def test_decode_step_equals_last_prefill_row_and_row_sampling():
    g = rng(7)
    S, H, Hkv, hd = 40, 4, 2, 128
    q = g.standard_normal((S, H, hd), dtype=np.float32)
    k = g.standard_normal((S, Hkv, hd), dtype=np.float32)
    v = g.standard_normal((S, Hkv, hd), dtype=np.float32)
    th = oracle.theta_table(hd, 5e5)
    full = oracle.attn_forward(q, k, v, oracle.SeqCache(S, Hkv, hd), theta=th, rope_mode=1)
    c = oracle.SeqCache(S, Hkv, hd)
    oracle.attn_forward(q[:S - 1], k[:S - 1], v[:S - 1], c, theta=th, rope_mode=1, rows=[[0, 0]])
    dec = oracle.attn_forward(q[S - 1:], k[S - 1:], v[S - 1:], c, theta=th, rope_mode=1)
    assert np.array_equal(dec[0], full[S - 1])  # same arithmetic, bit for bit
    rows = np.array([[3, 1], [39, 3], [0, 0]], np.int32)
    samp = oracle.attn_forward(q, k, v, oracle.SeqCache(S, Hkv, hd), theta=th, rope_mode=1, rows=rows)
    for r, (t, h) in enumerate(rows):
        assert np.array_equal(samp[r], full[t, h])
    # threads do not change results
    mt = oracle.attn_forward(q, k, v, oracle.SeqCache(S, Hkv, hd), theta=th, rope_mode=1, n_threads=4)
    assert np.array_equal(mt, full)


def test_fp16_rounding_is_rn_even_and_cache_variant():
    vals = np.array([1.0, 1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 1e-8, -2.5], np.float32)
    got = np.array([oracle.lib().hl_ref_round_fp16(float(x)) for x in vals], np.float32)
    assert np.array_equal(got, vals.astype(np.float16).astype(np.float32))
    assert got[1] == 1.0 and got[2] == np.float32(1.0 + 2 ** -9)  # ties to even both ways
    g = rng(8)
    S, H, Hkv, hd = 8, 2, 1, 64
    q = g.standard_normal((S, H, hd), dtype=np.float32)
    k = g.standard_normal((S, Hkv, hd), dtype=np.float32)
    v = g.standard_normal((S, Hkv, hd), dtype=np.float32)
    th = oracle.theta_table(hd, 1e4)
    c = oracle.SeqCache(S, Hkv, hd)
    oracle.attn_forward(q, k, v, c, theta=th, rope_mode=0, kv_fp16=True)
    assert np.array_equal(c.v, oracle.round_fp16(v))
    assert np.array_equal(c.k, oracle.round_fp16(c.k))


def test_bad_arguments_rejected():
    th = oracle.theta_table(64, 1e4)
    z = np.zeros((2, 3, 64), np.float32)
    kz = np.zeros((2, 2, 64), np.float32)
    with pytest.raises(ValueError):  # 3 heads not divisible by 2 kv heads
        oracle.attn_forward(z, kz, kz, oracle.SeqCache(4, 2, 64), theta=th, rope_mode=0)
    with pytest.raises(ValueError):  # cache too small
        oracle.attn_forward(np.zeros((2, 2, 64), np.float32), kz, kz, oracle.SeqCache(1, 2, 64), theta=th, rope_mode=0)
