"""The backend contract on a dense llama / qwen3 model (hl_dense_*): embedding, RMSNorm, Q/K/V/O projections,
SwiGLU FFN and vocabulary projection around the attention path, against the same layer stack written with
the oracle's tensor ops (matmul, rmsnorm, attention) -- the lkAttentionFfn branch of the reference's forward
pass (src/hippo_leap/backends/naive.nim:4054-4086).  Two oracles: plain float32 (loose tolerance: the CUDA path
feeds its GEMMs fp16 activations) and one that rounds activations to fp16 at the same points (tight)."""
import numpy as np
import pytest

import hippo_leap_b200 as hl
import oracle
from hippo_leap_b200 import dense as D
from tests.helpers import assert_parity, rel_l2

pytestmark = pytest.mark.gpu


class OracleDense:
    def __init__(self, m: D.DenseModel, max_len: int, mirror_fp16: bool, matmul=None):
        # matmul: the oracle's triple loop (tensor.nim:63-81) unless a test at large widths passes a faster stand-in
        self.mm = matmul or oracle.matmul
        hp = m.hparams
        self.m, self.hp, self.mirror = m, hp, mirror_fp16
        th = oracle.theta_table(hp.ropeDim or hp.headDim, hp.ropeFreqBase)
        self.theta = hl.theta_llama3_scale(th) if hp.llama3Scaling else th
        self.caches = [oracle.SeqCache(max_len, hp.nHeadKv, hp.headDim) for _ in range(hp.nLayer)]
        self.t = {k: np.ascontiguousarray(np.swapaxes(m.w[k].astype(np.float32), -1, -2))
                  for k in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down", "w_out")}

    def r(self, a):
        return oracle.round_fp16(a) if self.mirror else a

    def forward(self, tokens):
        hp, w, t = self.hp, self.m.w, self.t
        toks = np.asarray(tokens, np.int64)
        n = len(toks)
        x = w["tok_emb"][toks].astype(np.float32)
        for l in range(hp.nLayer):
            xn = self.r(oracle.rmsnorm(x, w["attn_norm"][l], hp.rmsEps))
            q = self.mm(xn, t["wq"][l]).reshape(n, hp.nHead, hp.headDim)
            k = self.mm(xn, t["wk"][l]).reshape(n, hp.nHeadKv, hp.headDim)
            v = self.mm(xn, t["wv"][l]).reshape(n, hp.nHeadKv, hp.headDim)
            o = oracle.attn_forward(q, k, v, self.caches[l], theta=self.theta, rope_mode=hp.ropeMode,
                                    q_norm_w=None if w["q_norm"] is None else w["q_norm"][l],
                                    k_norm_w=None if w["k_norm"] is None else w["k_norm"][l], eps=hp.rmsEps,
                                    kv_fp16=self.mirror)
            o = self.r(o.reshape(n, -1))
            x = (x + self.mm(o, t["wo"][l])).astype(np.float32)
            xn = self.r(oracle.rmsnorm(x, w["ffn_norm"][l], hp.rmsEps))
            g = self.r(self.mm(xn, t["w_gate"][l]))
            u = self.r(self.mm(xn, t["w_up"][l]))
            h = self.r((g / (1.0 + np.exp(-g))).astype(np.float32) * u)  # silu(x) = x / (1 + exp(-x)), tensor.nim silu
            x = (x + self.mm(h, t["w_down"][l])).astype(np.float32)
        xn = self.r(oracle.rmsnorm(x[-1:], w["out_norm"], hp.rmsEps))
        return self.mm(xn, t["w_out"])


CASES = {
    "llama_hd64": (D.DenseHParams(nVocab=512, nEmb=256, nLayer=2, nFfn=512, nHead=4, nHeadKv=2, headDim=64,
                                  ropeFreqBase=10000.0, rmsEps=1e-5, ropeMode=hl.HL_ROPE_SPLIT_HALF), False),
    "llama3_interleaved": (D.DenseHParams(nVocab=384, nEmb=256, nLayer=2, nFfn=768, nHead=4, nHeadKv=4, headDim=64,
                                          ropeFreqBase=500000.0, rmsEps=1e-5, ropeMode=hl.HL_ROPE_INTERLEAVED,
                                          llama3Scaling=True), False),
    "qwen3_hd128_qknorm": (D.DenseHParams(nVocab=640, nEmb=512, nLayer=3, nFfn=1024, nHead=4, nHeadKv=1, headDim=128,
                                          ropeFreqBase=1000000.0, rmsEps=1e-6, ropeMode=hl.HL_ROPE_SPLIT_HALF), True),
}


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("prompt_len,graph", [(5, True), (150, True), (3, False)])
def test_dense_model_against_oracle(name, prompt_len, graph):
    hp, qk_norm = CASES[name]
    D.setDecodeGraph(graph)
    steps, seed = 6, 11
    m = D.random_dense_model(hp, seed, qk_norm)
    max_len = prompt_len + steps + 2
    cache = D.initKvCache(hp, max_len)
    D.loadModelBackend(m, hp)
    plain, mirror = OracleDense(m, max_len, False), OracleDense(m, max_len, True)
    try:
        prompt = np.random.Generator(np.random.PCG64([seed, 1])).integers(0, hp.nVocab, prompt_len).astype(np.int32)
        cache.curLen = 0
        logits = D.forwardPrefill(m, prompt, cache)
        assert cache.curLen == prompt_len
        feed = prompt
        for step in range(steps + 1):
            # each step: both oracles and the CUDA path consume the same tokens (the oracle's greedy choice), so one
            # near-tie cannot end the comparison early; the argmax must agree wherever the margin is clear
            want, want_m = plain.forward(feed), mirror.forward(feed)
            scale = float(np.abs(want).max())
            top2 = np.sort(want_m[0])[-2:]
            clear = top2[1] - top2[0] > 1e-2 * scale
            tok = D.argmaxLast(want_m, hp.nVocab)
            if logits is not None:
                assert_parity(logits, want, f"step {step} logits vs float32 oracle", max_abs_tol=1e-2 * scale,
                              rel_l2_tol=5e-3)
                assert_parity(logits, want_m, f"step {step} logits vs fp16-activation oracle", max_abs_tol=3e-3 * scale,
                              rel_l2_tol=1.5e-3)
                got_tok = D.argmaxLast(logits, hp.nVocab)
            assert got_tok == tok or not clear, f"step {step}: token {got_tok}, oracle {tok}"
            if step == steps:
                break
            feed = [tok]
            if step % 2 == 0:
                logits = D.forwardDecode(m, tok, cache)
            else:
                logits = None
                got_tok, ms = D.forwardDecodeTokenTimed(m, tok, cache)
                assert ms > 0
            assert cache.curLen == prompt_len + step + 1
        assert cache.curLen <= max_len
    finally:
        D.unloadModelBackend()


def test_dense_llama32_1b_dimensions_one_layer():
    """One layer at the real Llama-3.2-1B widths (n_emb 2048, n_ffn 8192, 32 / 8 heads of 64, llama3-scaled theta) and
    a 32000-entry vocabulary: the SM-pair GEMM on the 520-token prompt, the split-K decode projections (K = 8192) and
    the two-stage argmax run at the sizes the benchmark uses.  At these widths the oracle's scalar triple loop takes
    minutes, so the same layer stack is evaluated with a float64 numpy contraction rounded to float32 (the small cases
    above pin the C oracle itself)."""
    hp = D.DenseHParams(nVocab=32000, nEmb=2048, nLayer=1, nFfn=8192, nHead=32, nHeadKv=8, headDim=64,
                        ropeFreqBase=500000.0, rmsEps=1e-5, ropeMode=hl.HL_ROPE_SPLIT_HALF, llama3Scaling=True)
    m = D.random_dense_model(hp, 31)
    prompt = np.random.Generator(np.random.PCG64([31, 1])).integers(0, hp.nVocab, 520).astype(np.int32)
    max_len = 528
    cache = D.initKvCache(hp, max_len)
    D.loadModelBackend(m, hp)
    ref = OracleDense(m, max_len, True, matmul=lambda a, b: (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))
    try:
        logits = D.forwardPrefill(m, prompt, cache)
        want = ref.forward(prompt)
        scale = float(np.abs(want).max())
        assert_parity(logits, want, "prefill logits", max_abs_tol=3e-3 * scale, rel_l2_tol=1.5e-3)
        tok = D.argmaxLast(want, hp.nVocab)
        for step in range(3):
            got_tok, ms = D.forwardDecodeTokenTimed(m, tok, cache)
            want = ref.forward([tok])
            top2 = np.sort(want[0])[-2:]
            tok = D.argmaxLast(want, hp.nVocab)
            assert got_tok == tok or top2[1] - top2[0] <= 1e-2 * float(np.abs(want).max()), f"step {step}"
        logits = D.forwardDecode(m, tok, cache)
        want = ref.forward([tok])
        assert_parity(logits, want, "decode logits", max_abs_tol=3e-3 * float(np.abs(want).max()), rel_l2_tol=1.5e-3)
    finally:
        D.unloadModelBackend()


def test_dense_graph_replay_equals_plain_launches():
    """The captured decode step and the same kernels queued one by one give bit-identical logits."""
    hp, qk_norm = CASES["qwen3_hd128_qknorm"]
    m = D.random_dense_model(hp, 4, qk_norm)
    cache = D.initKvCache(hp, 64)
    D.loadModelBackend(m, hp)
    try:
        prompt = np.arange(1, 31, dtype=np.int32)
        runs = []
        for graph in (True, False):
            D.setDecodeGraph(graph)
            cache.curLen = 0
            out = [D.forwardPrefill(m, prompt, cache)]
            tok = D.argmaxLast(out[0], hp.nVocab)
            for _ in range(5):
                out.append(D.forwardDecode(m, tok, cache))
                tok = D.argmaxLast(out[-1], hp.nVocab)
            runs.append(np.concatenate(out))
        assert np.array_equal(runs[0], runs[1])
    finally:
        D.setDecodeGraph(True)
        D.unloadModelBackend()


@pytest.mark.parametrize("name", ["llama_hd64", "qwen3_hd128_qknorm"])
def test_dense_chunked_prefill_and_prefix_reuse(name):
    """A prompt fed in pieces (positions continue at curLen) and a second prompt on a kept prefix, against the oracle
    fed the same way, and against the one-shot prefill."""
    hp, qk_norm = CASES[name]
    m = D.random_dense_model(hp, 21, qk_norm)
    g = np.random.Generator(np.random.PCG64([21, 1]))
    prefix, tail_a, tail_b = (g.integers(0, hp.nVocab, n).astype(np.int32) for n in (150, 77, 40))
    max_len = 150 + 77 + 8
    cache = D.initKvCache(hp, max_len)
    D.loadModelBackend(m, hp)
    try:
        one_shot = D.forwardPrefill(m, np.concatenate([prefix, tail_a]), cache)
        # chunked: 150 + 64 + 13, unequal pieces, the second and third start inside a 128-token page
        cache.curLen = 0
        D.forwardPrefillChunk(m, prefix, cache)
        D.forwardPrefillChunk(m, tail_a[:64], cache)
        chunked = D.forwardPrefillChunk(m, tail_a[64:], cache)
        assert cache.curLen == 227
        ref = OracleDense(m, max_len, True)
        ref.forward(prefix)
        ref.forward(tail_a[:64])
        want = ref.forward(tail_a[64:])
        scale = float(np.abs(want).max())
        assert_parity(chunked, want, "chunked prefill vs oracle", max_abs_tol=3e-3 * scale, rel_l2_tol=1.5e-3)
        assert_parity(chunked, one_shot, "chunked vs one-shot prefill", max_abs_tol=2e-3 * scale, rel_l2_tol=1e-3)
        # prefix reuse: keep the first 150 positions, replace what follows
        cache.curLen = 150
        reused = D.forwardPrefillChunk(m, tail_b, cache)
        assert cache.curLen == 190
        for c in ref.caches:
            c.cur_len = 150
        want_b = ref.forward(tail_b)
        assert_parity(reused, want_b, "prefix reuse vs oracle", max_abs_tol=3e-3 * float(np.abs(want_b).max()),
                      rel_l2_tol=1.5e-3)
        tok = D.argmaxLast(reused, hp.nVocab)
        nxt = D.forwardDecode(m, tok, cache)
        assert_parity(nxt, ref.forward([tok]), "decode after prefix reuse", max_abs_tol=3e-3 * scale, rel_l2_tol=1.5e-3)
        with pytest.raises(ValueError, match="exceeds KV cache capacity"):
            D.forwardPrefillChunk(m, np.zeros(max_len, np.int32), cache)
    finally:
        D.unloadModelBackend()


def test_dense_generate_loop_and_bench_cli(capsys):
    """The reference's generate loop and bench table (inference.nim:51-97, cmd_bench.nim:93-136) on the dense model."""
    from hippo_leap_b200 import backend as B
    from hippo_leap_b200 import cmd_bench
    hp, _ = CASES["llama_hd64"]
    m = D.random_dense_model(hp, 2)
    cache = D.initKvCache(hp, 64)
    D.loadModelBackend(m, hp)
    try:
        res = B.generate(m, cache, [1, 2, 3, 4, 5], 8, procs=D)
        assert res.completionTokens == 8 and res.gpuMs > 0 and cache.curLen == 5 + 7
        assert B.generate(m, cache, [1, 2, 3, 4, 5], 8, procs=D).tokens == res.tokens
    finally:
        D.freeKvCache(cache)
        D.unloadModelBackend()
    assert cmd_bench.main(["--model", "dense", "--config", "1", "--layers", "2", "--emb", "256", "--ffn", "512", "--vocab",
                           "1000", "--prompt-tokens", "20", "--tokens", "6", "--runs", "2", "--warmup", "1", "--context",
                           "64"]) == 0
    out = capsys.readouterr().out
    assert "dense layer stack" in out and " Run  Tokens  Time(ms)   tok/s   GPU(ms)  gpu tok/s" in out
    assert "Wall:" in out and "GPU :" in out


@pytest.mark.parametrize("name,graph", [("llama_hd64", True), ("qwen3_hd128_qknorm", True), ("llama_hd64", False)])
def test_batched_decode_of_several_sequences(name, graph):
    """hl_dense_batch_*: five sequences of different lengths in one page pool; every step decodes a different subset
    (5 rows: GEMV for up to 15 rows; 3 and 1: the fused decode projections; and a step after a prefix-reusing prefill).
    Each row must equal what that sequence gives alone through forwardPrefill / forwardDecode, and the oracle."""
    hp, qk_norm = CASES[name]
    m = D.random_dense_model(hp, 41, qk_norm)
    g = np.random.Generator(np.random.PCG64([41, 1]))
    lens = [3, 40, 129, 17, 260]
    prompts = [g.integers(0, hp.nVocab, n).astype(np.int32) for n in lens]
    max_len = 280
    D.setDecodeGraph(graph)   # a captured graph per number of active sequences, or plain launches
    D.loadModelBackend(m, hp)
    batch = D.DecodeBatch(m, 6, max_len)
    single = D.initKvCache(hp, max_len)
    try:
        refs, toks = [], []
        for s, p in enumerate(prompts):
            logits = batch.prefill(s, p)
            single.curLen = 0
            alone = D.forwardPrefill(m, p, single)
            assert np.array_equal(logits, alone), "prefill in the shared pool differs from the private cache"
            ref = OracleDense(m, max_len, True)
            want = ref.forward(p)
            assert_parity(logits, want, f"seq {s} prefill", max_abs_tol=3e-3 * float(np.abs(want).max()), rel_l2_tol=1.5e-3)
            refs.append(ref)
            toks.append(D.argmaxLast(want, hp.nVocab))
            assert batch.seq_len(s) == len(p)
        for step, active in enumerate([[0, 1, 2, 3, 4], [4, 2, 0], [1], [3, 0, 1, 2], [0, 1, 2, 3, 4]]):
            nxt, logits = batch.decode(active, [toks[s] for s in active], want_logits=True)
            for i, s in enumerate(active):
                want = refs[s].forward([toks[s]])
                scale = float(np.abs(want).max())
                assert_parity(logits[i:i + 1], want, f"step {step} seq {s}", max_abs_tol=3e-3 * scale, rel_l2_tol=1.5e-3)
                top2 = np.sort(want[0])[-2:]
                toks[s] = D.argmaxLast(want, hp.nVocab)
                assert nxt[i] == toks[s] or top2[1] - top2[0] <= 1e-2 * scale
        assert [batch.seq_len(s) for s in range(5)] == [lens[0] + 4, lens[1] + 4, lens[2] + 4, lens[3] + 3, lens[4] + 3]
        # the same step for one sequence alone, through the single-sequence contract on a private cache
        single.curLen = 0
        D.forwardPrefill(m, prompts[1], single)
        b2 = D.DecodeBatch(m, 2, max_len)
        b2.prefill(1, prompts[1])
        t0 = 7
        alone = D.forwardDecode(m, t0, single)
        _, together = b2.decode([1], [t0], want_logits=True)
        assert_parity(together, alone, "batch of one vs forwardDecode", max_abs_tol=1e-5 * float(np.abs(alone).max()) + 1e-6,
                      rel_l2_tol=1e-5)
        # prefix reuse inside the pool, then errors
        b2.prefill(1, prompts[3], start_pos=20)
        assert b2.seq_len(1) == 20 + lens[3]
        with pytest.raises(ValueError, match="twice"):
            b2.decode([1, 1], [1, 2])
        with pytest.raises(ValueError, match="out of range"):
            b2.decode([2], [1])
        with pytest.raises(ValueError, match="start_pos"):
            b2.prefill(0, prompts[0], start_pos=5)
        with pytest.raises(ValueError, match="exceeds KV cache capacity"):
            b2.prefill(0, np.zeros(max_len + 1, np.int32))
        b2.close()
    finally:
        D.setDecodeGraph(True)
        batch.close()
        D.freeKvCache(single)
        D.unloadModelBackend()


def test_decode_graphs_are_recaptured_when_buffers_grow():
    """A captured decode step holds the addresses of grow-only buffers.  A longer prompt (activations), a larger batch
    (split-KV and split-K scratch) re-allocate them; the next replay must run on the new ones."""
    hp, qk_norm = CASES["llama_hd64"]
    m = D.random_dense_model(hp, 51, qk_norm)
    g = np.random.Generator(np.random.PCG64([51, 1]))
    short, long_ = g.integers(0, hp.nVocab, 4).astype(np.int32), g.integers(0, hp.nVocab, 300).astype(np.int32)
    max_len = 320
    D.setDecodeGraph(True)
    cache = D.initKvCache(hp, max_len)
    D.loadModelBackend(m, hp)
    try:
        ref = OracleDense(m, max_len, True)
        for prompt in (short, long_, short):          # the long prompt re-allocates the activations between graph replays
            cache.curLen = 0
            for c in ref.caches:
                c.cur_len = 0
            want = ref.forward(prompt)
            assert_parity(D.forwardPrefill(m, prompt, cache), want, "prefill", max_abs_tol=3e-3 * float(np.abs(want).max()),
                          rel_l2_tol=1.5e-3)
            tok = D.argmaxLast(want, hp.nVocab)
            for _ in range(3):
                got, want = D.forwardDecode(m, tok, cache), ref.forward([tok])
                assert_parity(got, want, "decode", max_abs_tol=3e-3 * float(np.abs(want).max()), rel_l2_tol=1.5e-3)
                tok = D.argmaxLast(want, hp.nVocab)
        batch = D.DecodeBatch(m, 8, max_len)
        try:
            refs = [OracleDense(m, max_len, True) for _ in range(8)]
            toks = []
            for s_ in range(8):
                p_ = g.integers(0, hp.nVocab, 10 + 30 * s_).astype(np.int32)
                batch.prefill(s_, p_)
                toks.append(D.argmaxLast(refs[s_].forward(p_), hp.nVocab))
            for active in ([0], [1, 2], [0, 1, 2, 3, 4, 5, 6, 7], [0], [3, 1], [7, 6, 5, 4, 3, 2, 1, 0]):  # small graphs first
                _, logits = batch.decode(active, [toks[s_] for s_ in active], want_logits=True)
                for i, s_ in enumerate(active):
                    want = refs[s_].forward([toks[s_]])
                    assert_parity(logits[i:i + 1], want, f"batch {active} seq {s_}", max_abs_tol=3e-3 * float(np.abs(want).max()),
                                  rel_l2_tol=1.5e-3)
                    toks[s_] = D.argmaxLast(want, hp.nVocab)
        finally:
            batch.close()
    finally:
        D.unloadModelBackend()


def test_dense_older_cache_survives_larger_and_smaller_caches_created_after_it():
    """The identity block table is shared and grow-only: a larger cache re-allocates it (the older cache's decode graph
    must be captured again, not replayed through freed memory), a smaller one must not shorten the older cache's view."""
    hp, qk_norm = CASES["llama_hd64"]
    m = D.random_dense_model(hp, 61, qk_norm)
    g = np.random.Generator(np.random.PCG64([61, 1]))
    max_len = 420
    D.setDecodeGraph(True)
    cache_a = D.initKvCache(hp, max_len)
    D.loadModelBackend(m, hp)
    others = []
    try:
        ref = OracleDense(m, max_len, True)
        prompt = g.integers(0, hp.nVocab, 40).astype(np.int32)
        cache_a.curLen = 0
        want = ref.forward(prompt)
        assert_parity(D.forwardPrefill(m, prompt, cache_a), want, "prefill", max_abs_tol=3e-3 * float(np.abs(want).max()),
                      rel_l2_tol=1.5e-3)
        tok = D.argmaxLast(want, hp.nVocab)
        for step in range(8):
            if step == 4:
                others.append(D.initKvCache(hp, 4000))   # larger: the shared table moves
            got, want = D.forwardDecode(m, tok, cache_a), ref.forward([tok])
            assert_parity(got, want, f"decode step {step}", max_abs_tol=3e-3 * float(np.abs(want).max()), rel_l2_tol=1.5e-3)
            tok = D.argmaxLast(want, hp.nVocab)
        others.append(D.initKvCache(hp, 100))            # smaller: one 128-token block
        long_ = g.integers(0, hp.nVocab, 300).astype(np.int32)
        cache_a.curLen = 0
        for c in ref.caches:
            c.cur_len = 0
        want = ref.forward(long_)
        assert_parity(D.forwardPrefill(m, long_, cache_a), want, "prefill past the smaller cache's capacity",
                      max_abs_tol=3e-3 * float(np.abs(want).max()), rel_l2_tol=1.5e-3)
        tok = D.argmaxLast(want, hp.nVocab)
        got, want = D.forwardDecode(m, tok, cache_a), ref.forward([tok])
        assert_parity(got, want, "decode after it", max_abs_tol=3e-3 * float(np.abs(want).max()), rel_l2_tol=1.5e-3)
    finally:
        for c in others:
            D.freeKvCache(c)
        D.freeKvCache(cache_a)
        D.unloadModelBackend()


def test_dense_contract_errors():
    hp, _ = CASES["llama_hd64"]
    m = D.random_dense_model(hp, 3)
    with pytest.raises(ValueError, match="no model loaded"):
        D.forwardDecode(m, 1, D.KvCache())
    cache = D.initKvCache(hp, 8)
    D.loadModelBackend(m, hp)
    try:
        with pytest.raises(ValueError, match="already loaded"):
            D.loadModelBackend(m, hp)
        with pytest.raises(ValueError, match="exceeds KV cache capacity"):
            D.forwardPrefill(m, np.zeros(9, np.int32), cache)
        with pytest.raises(ValueError, match="at least one token"):
            D.forwardPrefill(m, np.zeros(0, np.int32), cache)
        D.forwardPrefill(m, np.arange(8, dtype=np.int32), cache)
        with pytest.raises(ValueError, match="KV cache full"):
            D.forwardDecode(m, 1, cache)
    finally:
        D.unloadModelBackend()
    bad = D.DenseHParams(nVocab=64, nEmb=64, nLayer=1, nFfn=64, nHead=3, nHeadKv=2, headDim=64)
    with pytest.raises(ValueError, match="divisible"):
        D.initKvCache(bad, 8)
