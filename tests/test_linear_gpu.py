"""The dense fp16 projection (hl_b200_linear_f16) against the oracle's matmul (tensor.nim:63-81) on the
fp16-rounded operands: tcgen05 GEMM for prefill-sized M, GEMV for decode-sized M, ragged edges, residual,
and the attention -> output-projection hand-off in fp16."""
import numpy as np
import pytest
import torch

import hippo_leap_b200 as hl
import oracle

pytestmark = pytest.mark.gpu


def _check(hl_ctx, M, N, K, resid, out_dtype, seed=0):
    g = np.random.Generator(np.random.PCG64([seed, M, N, K]))
    a = g.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    w = (g.standard_normal((N, K), dtype=np.float32) / np.sqrt(K)).astype(np.float16)
    r = g.standard_normal((M, N), dtype=np.float32) if resid else None
    out = hl_ctx.linear_f16(torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda(),
                            resid=None if r is None else torch.from_numpy(r).cuda(), out_dtype=out_dtype)
    got = out.float().cpu().numpy()
    want = oracle.matmul(a.astype(np.float32), np.ascontiguousarray(w.astype(np.float32).T))
    if r is not None:
        want = want + r
    tol = 2e-3 if out_dtype == torch.float16 else 2e-4 * max(1.0, np.sqrt(K / 256))
    err = float(np.abs(got - want).max())
    assert err < tol * max(1.0, float(np.abs(want).max())), f"M={M} N={N} K={K}: max-abs {err:.3e}"
    assert hl_ctx.device_status() == (0, 0)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 128), (2048, 2048, 2048), (200, 300, 72),
                                   (17, 5, 8), (1000, 256, 4096), (129, 257, 200)])
def test_gemm_against_oracle_matmul(hl_ctx, M, N, K):
    _check(hl_ctx, M, N, K, resid=False, out_dtype=torch.float32)


@pytest.mark.parametrize("M,N,K", [(1, 2048, 2048), (3, 512, 1000), (8, 130, 64), (15, 64, 4096)])
def test_gemv_against_oracle_matmul(hl_ctx, M, N, K):
    _check(hl_ctx, M, N, K, resid=True, out_dtype=torch.float32)


@pytest.mark.parametrize("M,N,K,resid,dt", [
    (2, 64, 32, False, torch.float32),          # two rows padded to 16, one K step
    (5, 64, 32, False, torch.float32),
    (9, 3072, 2048, False, torch.float32),      # Q|K|V shape, eight splits
    (12, 128, 8200, True, torch.float16),       # K not a multiple of 64: the TMA box past the end is zero
    (16, 2048, 2048, True, torch.float32),      # split-K, partials added by the reduction kernel
    (17, 300, 200, True, torch.float16),        # 32-row padding, ragged N and K
    (33, 1000, 4096, False, torch.float32),     # 64-row padding
    (64, 2048, 8192, True, torch.float32),      # the down projection of a 64-sequence step
    (40, 16384, 2048, False, torch.float16),    # gate|up shape: no split
])
def test_several_row_projection_against_oracle_matmul(hl_ctx, M, N, K, resid, dt):
    """2 <= M <= 128 runs on tcgen05 with W on the M side of the MMA and split-K for short N (linear_wide.cuh); twice
    in a row on different data, so that stale split-K partials would show."""
    _check(hl_ctx, M, N, K, resid=resid, out_dtype=dt, seed=M + N)
    _check(hl_ctx, M, N, K, resid=resid, out_dtype=dt, seed=M + N + 1)


@pytest.mark.parametrize("M,N,K,resid,dt", [
    (512, 256, 64, False, torch.float32),       # one pair tile per 256 columns, a single K step
    (600, 300, 200, True, torch.float32),       # ragged in M (the peer CTA's last rows), N and K
    (4096, 1024, 512, False, torch.float16),    # more tiles than SM pairs: both accumulators, ring wrap-around
    (769, 513, 1032, True, torch.float16),      # second CTA of the last pair row holds a single live row
])
def test_pair_gemm_against_oracle_matmul(hl_ctx, M, N, K, resid, dt):
    """M >= 512 runs on SM pairs (256 x 256 tiles, tcgen05 cta_group::2)."""
    _check(hl_ctx, M, N, K, resid=resid, out_dtype=dt, seed=M + N)


def test_residual_and_fp16_output(hl_ctx):
    _check(hl_ctx, 384, 512, 256, resid=True, out_dtype=torch.float32, seed=3)
    _check(hl_ctx, 384, 512, 256, resid=False, out_dtype=torch.float16, seed=4)


def test_attention_output_feeds_the_projection_in_fp16(hl_ctx):
    """fp16 attention output, token-major [S, n_head*hd], straight into the Wo GEMM (naive.nim:4079)."""
    from hippo_leap_b200 import synth
    from tests.helpers import oracle_seq
    cfg = synth.CONFIGS[1]
    S, bt, n_emb = 256, 16, 512
    q, k, v = synth.gen_qkv(cfg, S)
    theta = cfg.theta()
    hl_ctx.set_rope(theta)
    shape = hl.AttnShape(cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.head_dim, hl.HL_ROPE_SPLIT_HALF)
    tq, tk, tv = (torch.from_numpy(x).cuda() for x in (q, k, v))
    tt = torch.arange(S // bt, dtype=torch.int32, device="cuda")
    kv = hl_ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, S // bt)
    hl_ctx.kv_append_seq(kv, 0, shape, tk, tv, 0, tt)
    attn16 = torch.empty((S, cfg.n_head, cfg.head_dim), dtype=torch.float16, device="cuda")
    hl_ctx.attn_prefill(kv, 0, shape, tq, 0, tt, attn16)
    g = np.random.Generator(np.random.PCG64(5))
    wo = (g.standard_normal((n_emb, cfg.n_head * cfg.head_dim), dtype=np.float32) / 45).astype(np.float16)
    got = hl_ctx.linear_f16(attn16.view(S, -1), torch.from_numpy(wo).cuda()).cpu().numpy()
    ref_attn = oracle_seq(q, k, v, theta=theta, rope_mode=1).reshape(S, -1)
    want = oracle.matmul(ref_attn, np.ascontiguousarray(wo.astype(np.float32).T))
    assert float(np.abs(got - want).max()) < 5e-3 and float(np.linalg.norm(got - want) / np.linalg.norm(want)) < 2e-3
    kv.destroy()


@pytest.mark.parametrize("M,N,K", [(16, 64, 64), (100, 300, 200), (129, 512, 128), (300, 1024, 2048), (512, 512, 256),
                                   (640, 1100, 320), (2048, 1024, 512)])
def test_gate_up_projection_with_silu_in_the_epilogue(hl_ctx, M, N, K):
    """hl_b200_linear_f16_silu: h[m][c] = fp16(silu(gate) * up) with gate / up = accumulator columns 2c / 2c + 1
    (siluMulKernel, naive.nim:2179-2197, on the output of the merged projection).  Against the oracle's matmul on
    the fp16-rounded operands; and, where the plain projection runs the same GEMM kernel (M > 128), against the
    two-step form built from its fp16 output: equal up to one fp16 ulp where expf differs in its last bit."""
    g = np.random.Generator(np.random.PCG64([7, M, N, K]))
    a = g.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    w = (g.standard_normal((N, K), dtype=np.float32) / np.sqrt(K)).astype(np.float16)
    a_d, w_d = torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda()
    h = hl_ctx.linear_f16_silu(a_d, w_d)
    assert hl_ctx.device_status() == (0, 0)
    gu = oracle.matmul(a.astype(np.float32), np.ascontiguousarray(w.astype(np.float32).T)).astype(np.float16).astype(np.float32)
    gate, up = gu[:, 0::2], gu[:, 1::2]
    want = (gate / (1.0 + np.exp(-gate)) * up).astype(np.float32)
    got = h.float().cpu().numpy()
    assert got.shape == (M, N // 2)
    err = float(np.abs(got - want).max())
    assert err < 4e-3 * max(1.0, float(np.abs(want).max())), f"M={M} N={N} K={K}: max-abs {err:.3e} vs the oracle"
    if M > 128:
        gu_d = hl_ctx.linear_f16(a_d, w_d, out_dtype=torch.float16).float()
        two_step = (gu_d[:, 0::2] * torch.sigmoid(gu_d[:, 0::2]) * gu_d[:, 1::2]).half()
        diff = (h.view(torch.int16).int() - two_step.view(torch.int16).int()).abs()
        assert int(diff.max()) <= 1, "more than one fp16 ulp from the two-step form"
        assert float((diff != 0).float().mean()) < 2e-2


def test_gate_up_projection_refuses_what_it_cannot_do(hl_ctx):
    a = torch.zeros((8, 64), dtype=torch.float16, device="cuda")
    w = torch.zeros((64, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(hl.HlError):
        hl_ctx.linear_f16_silu(a, w)            # fewer than 16 rows: the decode path's fused GEMV serves those
    a = torch.zeros((32, 64), dtype=torch.float16, device="cuda")
    w = torch.zeros((63, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(hl.HlError):
        hl_ctx.linear_f16_silu(a, w, torch.empty((32, 31), dtype=torch.float16, device="cuda"))  # odd N
    assert hl_ctx.device_status() == (0, 0)


def test_projection_reproduces_the_reference_tests_known_answers(hl_ctx, wmma_known_answers):
    """The closed-form fp16 x fp16 -> fp32 products of the reference's tests/integration_wmma.nim (:33-60 and :70-76),
    through hl_b200_linear_f16 (out = A . W^T): exact, every value is an integer below 2^24."""
    for a, b, c in wmma_known_answers:
        w = np.ascontiguousarray(b.T)                          # W[n][k] = B[k][n]
        for rows in (16, 1):                                   # 16 rows: tcgen05 path; one row: the GEMV
            if w.shape[0] < 1:
                continue
            out = hl_ctx.linear_f16(torch.from_numpy(a[:rows].astype(np.float16)).cuda(),
                                    torch.from_numpy(w.astype(np.float16)).cuda())
            assert np.array_equal(out.cpu().numpy(), c[:rows]), (rows, out.cpu().numpy(), c[:rows])
    assert hl_ctx.device_status() == (0, 0)


def _random_gemm_cases(n, seed, budget):
    g = np.random.Generator(np.random.PCG64(seed))
    out = []
    while len(out) < n:
        M = int(g.choice([1, 2, 3, 4, 5, 15, 16, 17, 64, 127, 128, 129, 200, 511, 512, 513, 700]))
        N = int(g.choice([1, 8, 24, 100, 256, 257, 1000, 2048, 3072]))
        K = int(8 * g.integers(1, 600))
        if M * N * K > budget:
            continue
        out.append(pytest.param(M, N, K, bool(g.random() < 0.5), bool(g.random() < 0.4), len(out),
                                id=f"{len(out)}-{M}x{N}x{K}"))
    return out


@pytest.mark.parametrize("M,N,K,resid,half_out,seed", _random_gemm_cases(30, 20260103, 6e7))
def test_random_projection_shapes_against_oracle_matmul(hl_ctx, M, N, K, resid, half_out, seed):
    """Ragged M / N / K across the four kernels behind hl_b200_linear_f16 (GEMV, several-row, single-SM and SM-pair
    GEMM), with and without the residual, float32 or fp16 output."""
    _check(hl_ctx, M, N, K, resid=resid, out_dtype=torch.float16 if half_out else torch.float32, seed=1000 + seed)
