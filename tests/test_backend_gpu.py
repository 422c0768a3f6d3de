"""The reference's drive pattern (tests/integration_inference.nim:34-46) through the backend contract:
reset curLen, one prefill, argmax, N decode steps feeding the argmax back; the token id stream from
the CUDA path must equal the oracle's, and the contract's errors must match the reference's."""
import numpy as np
import pytest

import hippo_leap_b200 as hl
import oracle
from hippo_leap_b200 import backend as B
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu


class OracleModel:
    """CPU restatement of the stand-in model on top of the oracle's attention path."""

    def __init__(self, m: B.Model, max_len: int, rope_mode: int):
        hp = m.hparams
        self.m, self.hp, self.mode = m, hp, rope_mode
        th = oracle.theta_table(hp.ropeDim or hp.headDim, hp.ropeFreqBase)
        self.theta = hl.theta_llama3_scale(th) if hp.llama3Scaling else th
        self.caches = [oracle.SeqCache(max_len, hp.nHeadKv, hp.headDim) for _ in range(hp.nLayer)]

    def reset(self):
        for c in self.caches:
            c.cur_len = 0

    def forward(self, tokens):
        hp, m = self.hp, self.m
        toks = np.asarray(tokens, np.int64)
        x = None
        for l in range(hp.nLayer):
            q = m.eq[l][toks].reshape(len(toks), hp.nHead, hp.headDim)
            k = m.ek[l][toks].reshape(len(toks), hp.nHeadKv, hp.headDim)
            v = m.ev[l][toks].reshape(len(toks), hp.nHeadKv, hp.headDim)
            rows = np.array([[len(toks) - 1, h] for h in range(hp.nHead)], np.int32)
            o = oracle.attn_forward(q, k, v, self.caches[l], theta=self.theta, rope_mode=self.mode,
                                    q_norm_w=None if m.qNorm is None else m.qNorm[l],
                                    k_norm_w=None if m.kNorm is None else m.kNorm[l], eps=hp.rmsEps, rows=rows)
            o = o.reshape(-1)
            x = o if x is None else (x + o).astype(np.float32)
        return oracle.matmul(x[None, :], m.wout)  # [1, nVocab]


def _drive(hp, qk_norm, prompt_len, steps, seed):
    m = B.standin_model(hp, seed, qk_norm)
    max_len = prompt_len + steps + 3
    cache = B.initKvCache(hp, max_len)
    B.loadModelBackend(m, hp)
    ref = OracleModel(m, max_len, hp.ropeMode)
    try:
        prompt = np.random.Generator(np.random.PCG64([seed, 1])).integers(0, hp.nVocab, prompt_len).astype(np.int32)
        cache.curLen = 0
        logits = B.forwardPrefill(m, prompt, cache)
        want = ref.forward(prompt)
        assert cache.curLen == prompt_len
        assert_parity(logits, want, "prefill logits", max_abs_tol=2e-3 * float(np.abs(want).max()), rel_l2_tol=1e-3)
        tok, rtok = B.argmaxLast(logits, hp.nVocab), B.argmaxLast(want, hp.nVocab)
        got_stream, want_stream, margins = [tok], [rtok], []
        for i in range(steps):
            if i % 3 == 0:
                logits = B.forwardDecode(m, tok, cache)
                tok = B.argmaxLast(logits, hp.nVocab)
            elif i % 3 == 1:
                tok = B.forwardDecodeToken(m, tok, cache)
            else:
                tok, ms = B.forwardDecodeTokenTimed(m, tok, cache)
                assert ms > 0
            want = ref.forward([rtok])
            top2 = np.sort(want[0])[-2:]
            margins.append(float(top2[1] - top2[0]))
            rtok = B.argmaxLast(want, hp.nVocab)
            got_stream.append(tok)
            want_stream.append(rtok)
            if tok != rtok:
                break
        assert got_stream == want_stream, (
            f"greedy stream diverged at step {len(got_stream) - 1}: got {got_stream[-1]}, oracle {want_stream[-1]}, "
            f"oracle top-2 margin {margins[-1]:.3e}")
        assert cache.curLen == prompt_len + steps
        return m, cache
    except BaseException:
        B.freeKvCache(cache)
        B.unloadModelBackend()
        raise


def test_greedy_stream_config1_tinyllama_shape():
    """Config 1: 32/4 heads, hd 64, theta 1e4, 128-token prompt, 32 greedy steps, split-half RoPE (the
    pairing of the reference GPU backends whose token stream the drop-in must reproduce)."""
    hp = B.HParams(nVocab=512, nLayer=1, nHead=32, nHeadKv=4, headDim=64, ropeFreqBase=1e4)
    m, cache = _drive(hp, False, 128, 32, seed=0)
    # contract errors, as the reference raises them
    with pytest.raises(ValueError, match="at least one token"):
        B.forwardPrefill(m, [], cache)
    with pytest.raises(ValueError, match="exceeds KV cache capacity"):
        B.forwardPrefill(m, np.zeros(cache.maxLen + 1, np.int32), cache)
    cache.curLen = cache.maxLen
    with pytest.raises(ValueError, match="KV cache full"):
        B.forwardDecode(m, 1, cache)
    # an external reset of curLen starts a new request (inference.nim:58)
    cache.curLen = 0
    a = B.forwardPrefill(m, [5, 6, 7], cache)
    cache.curLen = 0
    b = B.forwardPrefill(m, [5, 6, 7], cache)
    assert np.array_equal(a, b) and cache.curLen == 3
    assert B.launchCount() > 0
    B.freeKvCache(cache)
    B.unloadModelBackend()
    with pytest.raises(ValueError, match="no model loaded"):
        B.forwardDecode(m, 1, cache)


def test_greedy_stream_interleaved_rope_tensor_nim_pairing():
    """Same drive with the CPU op's interleaved pairing (tensor.nim:156-166)."""
    hp = B.HParams(nVocab=512, nLayer=1, nHead=32, nHeadKv=4, headDim=64, ropeFreqBase=1e4,
                   ropeMode=hl.HL_ROPE_INTERLEAVED)
    m, cache = _drive(hp, False, 128, 32, seed=3)
    B.freeKvCache(cache)
    B.unloadModelBackend()


def test_greedy_stream_multilayer_llama3_scaled_theta_and_qk_norm():
    """Several layers, llama3-scaled theta, hd 128 with QK-norm: 4 layers, 300-token prompt, 40 steps."""
    hp = B.HParams(nVocab=512, nLayer=4, nHead=16, nHeadKv=4, headDim=128, ropeFreqBase=5e5, llama3Scaling=True)
    m, cache = _drive(hp, True, 300, 40, seed=5)
    B.freeKvCache(cache)
    B.unloadModelBackend()


def test_greedy_stream_head_dim_256_qwen35moe_attention_shape():
    """The attention shape of the reference's qwen35moe models (tests/integration_qwen36moe.nim:25-27: 16 / 2 heads,
    head_dim 256) through the contract: 2 layers, QK-norm, 270-token prompt, 24 steps."""
    hp = B.HParams(nVocab=512, nLayer=2, nHead=16, nHeadKv=2, headDim=256, ropeFreqBase=1e6)
    m, cache = _drive(hp, True, 270, 24, seed=9)
    B.freeKvCache(cache)
    B.unloadModelBackend()


def test_bad_hparams_rejected_before_any_launch():
    hp = B.HParams(nVocab=64, nLayer=1, nHead=6, nHeadKv=4, headDim=64)
    with pytest.raises(ValueError, match="divisible"):
        B.initKvCache(hp, 32)
    hp = B.HParams(nVocab=64, nLayer=1, nHead=4, nHeadKv=4, headDim=96)
    with pytest.raises(ValueError, match="head_dim"):
        B.initKvCache(hp, 32)
    B.unloadModelBackend()


def test_generate_loop_and_bench_cli(capsys):
    """generate() follows the reference loop (inference.nim:51-97) and the bench command prints the
    reference's table (cmd_bench.nim:101-136)."""
    from hippo_leap_b200 import cmd_bench
    hp = B.HParams(nVocab=512, nLayer=2, nHead=8, nHeadKv=2, headDim=64)
    m = B.standin_model(hp, 9)
    cache = B.initKvCache(hp, 64)
    B.loadModelBackend(m, hp)
    try:
        res = B.generate(m, cache, [1, 2, 3, 4], 8)
        assert res.promptTokens == 4 and res.completionTokens == 8 and res.totalTokens == 12
        assert res.elapsedMs > 0 and res.gpuMs > 0 and cache.curLen == 4 + 7
        again = B.generate(m, cache, [1, 2, 3, 4], 8)
        assert again.tokens == res.tokens                      # curLen reset -> same request, same stream
        assert B.generate(m, cache, [], 8).completionTokens == 0
        assert B.generate(m, cache, list(range(64)), 8).completionTokens == 0   # no room left in the context
        stop = res.tokens[2]
        assert B.generate(m, cache, [1, 2, 3, 4], 8, stopTokenIds=(stop,)).tokens == res.tokens[:res.tokens.index(stop) + 1]
    finally:
        B.freeKvCache(cache)
        B.unloadModelBackend()
    assert cmd_bench.main(["--config", "1", "--prompt-tokens", "32", "--tokens", "8", "--runs", "2", "--warmup", "1",
                           "--context", "64"]) == 0
    out = capsys.readouterr().out
    assert " Run  Tokens  Time(ms)   tok/s   GPU(ms)  gpu tok/s" in out
    assert "Wall:" in out and "GPU :" in out and "±" in out


def test_decode_graph_replay_equals_plain_launches():
    """forwardDecodeToken through the captured CUDA graph and through plain launches give the same ids,
    across a reset of curLen and a second cache (the graph is re-captured for another cache)."""
    hp = B.HParams(nVocab=512, nLayer=3, nHead=16, nHeadKv=4, headDim=128, ropeFreqBase=5e5)
    m = B.standin_model(hp, 12)
    cache = B.initKvCache(hp, 200)
    B.loadModelBackend(m, hp)
    try:
        prompt = list(range(7, 7 + 90))
        streams = {}
        for mode in (True, False, True):
            B.setDecodeGraph(mode)
            res = B.generate(m, cache, prompt, 60)
            streams.setdefault(mode, []).append(res.tokens)
        assert streams[True][0] == streams[False][0] == streams[True][1]
        cache2 = B.initKvCache(hp, 120)
        B.setDecodeGraph(True)
        assert B.generate(m, cache2, prompt, 25).tokens == streams[True][0][:25]
        B.freeKvCache(cache2)
    finally:
        B.setDecodeGraph(True)
        B.freeKvCache(cache)
        B.unloadModelBackend()


def test_chunked_prefill_and_prefix_reuse_stand_in_model():
    """forwardPrefillChunk: a prompt fed in pieces whose positions continue at curLen (RoPE at pos + p, a causal mask
    that is not square), and a new tail on a kept prefix; the oracle is driven the same way."""
    hp = B.HParams(nVocab=512, nLayer=2, nHead=16, nHeadKv=4, headDim=128, ropeFreqBase=1e6)
    m = B.standin_model(hp, 9, True)
    g = np.random.Generator(np.random.PCG64([9, 1]))
    prefix, tail_a, tail_b = (g.integers(0, hp.nVocab, n).astype(np.int32) for n in (200, 130, 33))
    max_len = 340
    cache = B.initKvCache(hp, max_len)
    B.loadModelBackend(m, hp)
    try:
        ref = OracleModel(m, max_len, hp.ropeMode)
        cache.curLen = 0
        B.forwardPrefillChunk(m, prefix, cache)
        B.forwardPrefillChunk(m, tail_a[:1], cache)  # a one-token piece goes through the prefill kernels too
        got = B.forwardPrefillChunk(m, tail_a[1:], cache)
        assert cache.curLen == 330
        ref.forward(prefix)
        ref.forward(tail_a[:1])
        want = ref.forward(tail_a[1:])
        assert_parity(got, want, "chunked prefill", max_abs_tol=2e-3 * float(np.abs(want).max()), rel_l2_tol=1e-3)
        cache.curLen = 0
        one_shot = B.forwardPrefill(m, np.concatenate([prefix, tail_a]), cache)
        assert_parity(got, one_shot, "chunked vs one-shot", max_abs_tol=2e-3 * float(np.abs(want).max()), rel_l2_tol=1e-3)
        cache.curLen = 200
        for c in ref.caches:
            c.cur_len = 200
        got_b, want_b = B.forwardPrefillChunk(m, tail_b, cache), ref.forward(tail_b)
        assert cache.curLen == 233
        assert_parity(got_b, want_b, "prefix reuse", max_abs_tol=2e-3 * float(np.abs(want_b).max()), rel_l2_tol=1e-3)
        with pytest.raises(ValueError, match="exceeds KV cache capacity"):
            B.forwardPrefillChunk(m, np.zeros(200, np.int32), cache)
    finally:
        B.freeKvCache(cache)
        B.unloadModelBackend()


def test_decode_graph_is_recaptured_when_a_longer_prompt_grows_the_buffers():
    """The captured decode step holds the addresses of the grow-only activation buffers; a longer prompt re-allocates
    them, and the next replay must use the new ones."""
    hp = B.HParams(nVocab=512, nLayer=2, nHead=8, nHeadKv=2, headDim=64)
    m = B.standin_model(hp, 17)
    max_len = 400
    cache = B.initKvCache(hp, max_len)
    B.loadModelBackend(m, hp)
    B.setDecodeGraph(True)
    try:
        ref = OracleModel(m, max_len, hp.ropeMode)
        g = np.random.Generator(np.random.PCG64([17, 1]))
        for n in (3, 350, 6):
            prompt = g.integers(0, hp.nVocab, n).astype(np.int32)
            cache.curLen = 0
            ref.reset()
            want = ref.forward(prompt)
            assert_parity(B.forwardPrefill(m, prompt, cache), want, "prefill", max_abs_tol=2e-3 * float(np.abs(want).max()),
                          rel_l2_tol=1e-3)
            tok = B.argmaxLast(want, hp.nVocab)
            for _ in range(4):
                got = B.forwardDecodeToken(m, tok, cache)
                want = ref.forward([tok])
                top2 = np.sort(want[0])[-2:]
                tok = B.argmaxLast(want, hp.nVocab)
                assert got == tok or top2[1] - top2[0] < 1e-3 * float(np.abs(want).max())
    finally:
        B.freeKvCache(cache)
        B.unloadModelBackend()


def test_an_older_cache_survives_larger_and_smaller_caches_created_after_it():
    """All caches share one grow-only identity block table.  A larger cache re-allocates it: the decode graph captured
    for the older cache must not replay through the freed table.  A smaller cache must not shorten the older cache's
    view of the table: a prompt past the smaller cache's capacity still fits the older one."""
    hp = B.HParams(nVocab=512, nLayer=2, nHead=8, nHeadKv=2, headDim=64)
    m = B.standin_model(hp, 21)
    cache_a = B.initKvCache(hp, 400)
    B.loadModelBackend(m, hp)
    others = []
    try:
        prompt = np.random.Generator(np.random.PCG64([21, 1])).integers(0, hp.nVocab, 90).astype(np.int32)
        B.setDecodeGraph(False)
        want = B.generate(m, cache_a, prompt, 40).tokens
        B.setDecodeGraph(True)
        cache_a.curLen = 0
        tok = B.argmaxLast(B.forwardPrefill(m, prompt, cache_a), hp.nVocab)
        got = [tok]
        for _ in range(19):
            tok = B.forwardDecodeToken(m, tok, cache_a)
            got.append(tok)
        others.append(B.initKvCache(hp, 3000))          # larger: the shared table is re-allocated
        for _ in range(20):
            tok = B.forwardDecodeToken(m, tok, cache_a)  # graph of cache A must have been captured again
            got.append(tok)
        assert got == want[:40]
        others.append(B.initKvCache(hp, 64))            # smaller: 4 blocks
        long_prompt = np.random.Generator(np.random.PCG64([21, 2])).integers(0, hp.nVocab, 300).astype(np.int32)
        ref = OracleModel(m, 400, hp.ropeMode)
        cache_a.curLen = 0
        logits, ref_logits = B.forwardPrefill(m, long_prompt, cache_a), ref.forward(long_prompt)
        assert_parity(logits, ref_logits, "prefill past the smaller cache's capacity",
                      max_abs_tol=2e-3 * float(np.abs(ref_logits).max()), rel_l2_tol=1e-3)
        tok = B.argmaxLast(ref_logits, hp.nVocab)
        got_tok, ref_next = B.forwardDecodeToken(m, tok, cache_a), ref.forward([tok])
        top2 = np.sort(ref_next[0])[-2:]
        assert got_tok == B.argmaxLast(ref_next, hp.nVocab) or top2[1] - top2[0] < 1e-3 * float(np.abs(ref_next).max())
    finally:
        B.setDecodeGraph(True)
        for c in others:
            B.freeKvCache(c)
        B.freeKvCache(cache_a)
        B.unloadModelBackend()
