"""The reference's backend contract, same names and meaning, over ``libhl_b200.so``.

hippo_leap picks a backend module at compile time (src/hippo_leap/inference.nim:7-14) and
calls ``initKvCache / loadModelBackend / unloadModelBackend / forwardPrefill / forwardDecode /
forwardDecodeToken / forwardDecodeTokenTimed`` on it.  This module is the testable mirror of
``src/hippo_leap/backends/b200.nim``: every function binds the ``hl_backend_*`` entry point
that the Nim proc of the same name binds, with the same argument order and error behaviour
(``ValueError`` for bad shapes, an empty prompt, a prompt beyond the cache, a full cache --
src/hippo_leap/backends/naive.nim:3969-3976, 4594-4599).

The model is the attention-only stand-in described in ``include/hl_backend.h``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib as L


class HParamsC(C.Structure):
    _fields_ = [("n_vocab", C.c_int32), ("n_layer", C.c_int32), ("n_head", C.c_int32),
                ("n_head_kv", C.c_int32), ("head_dim", C.c_int32), ("rope_dim", C.c_int32),
                ("rope_freq_base", C.c_float), ("rms_eps", C.c_float), ("rope_mode", C.c_int32),
                ("llama3_scaling", C.c_int32)]


class WeightsC(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("eq", "ek", "ev", "wout", "q_norm", "k_norm")]


class KvCacheC(C.Structure):
    _fields_ = [("cur_len", C.c_int32), ("max_len", C.c_int32), ("n_head_kv", C.c_int32),
                ("head_dim", C.c_int32), ("gpu_cache", C.c_void_p)]


_f32p, _i32 = C.POINTER(C.c_float), C.c_int32
BACKEND_SYMBOLS = {
    "hl_backend_init_kv_cache": (_i32, [_i32, C.POINTER(HParamsC), _i32, C.POINTER(KvCacheC)]),
    "hl_backend_free_kv_cache": (_i32, [C.POINTER(KvCacheC)]),
    "hl_backend_load_model": (_i32, [_i32, C.POINTER(HParamsC), C.POINTER(WeightsC)]),
    "hl_backend_unload_model": (_i32, []),
    "hl_backend_forward_prefill": (_i32, [C.POINTER(_i32), _i32, C.POINTER(KvCacheC), _f32p]),
    "hl_backend_forward_prefill_chunk": (_i32, [C.POINTER(_i32), _i32, C.POINTER(KvCacheC), _f32p]),
    "hl_backend_forward_decode": (_i32, [_i32, C.POINTER(KvCacheC), _f32p]),
    "hl_backend_forward_decode_token": (_i32, [_i32, C.POINTER(KvCacheC), C.POINTER(_i32)]),
    "hl_backend_forward_decode_token_timed": (_i32, [_i32, C.POINTER(KvCacheC), C.POINTER(_i32), _f32p]),
    "hl_backend_set_decode_graph": (_i32, [_i32]),
    "hl_backend_last_error": (C.c_char_p, []),
    "hl_backend_launch_count": (C.c_int64, []),
}
_typed = False


def _lib():
    global _typed
    lib = L.load()
    if not _typed:
        for name, (res, args) in BACKEND_SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _typed = True
    return lib


def _check(rc: int):
    if rc != 0:
        raise ValueError(f"{L.STATUS_NAMES.get(rc, rc)}: {_lib().hl_backend_last_error().decode()}")


@dataclass
class HParams:
    """The fields of HParams (src/hippo_leap/model.nim:24-50) that parameterise the path."""
    nVocab: int
    nLayer: int
    nHead: int
    nHeadKv: int
    headDim: int
    ropeDim: int = 0
    ropeFreqBase: float = 10000.0
    rmsEps: float = 1e-6
    ropeMode: int = L.HL_ROPE_SPLIT_HALF
    llama3Scaling: bool = False

    def c(self) -> HParamsC:
        return HParamsC(self.nVocab, self.nLayer, self.nHead, self.nHeadKv, self.headDim, self.ropeDim,
                        self.ropeFreqBase, self.rmsEps, self.ropeMode, int(self.llama3Scaling))


@dataclass
class Model:
    """Stand-in for the reference's Model: hparams + host float32 weights."""
    hparams: HParams
    eq: np.ndarray       # [nLayer, nVocab, nHead*headDim]
    ek: np.ndarray       # [nLayer, nVocab, nHeadKv*headDim]
    ev: np.ndarray
    wout: np.ndarray     # [nHead*headDim, nVocab]
    qNorm: np.ndarray | None = None   # [nLayer, headDim]
    kNorm: np.ndarray | None = None


def standin_model(hp: HParams, seed: int, qk_norm: bool = False) -> Model:
    """Seeded N(0,1) tables; gamma ~ U(0.9, 1.1) when qk_norm."""
    g = np.random.Generator(np.random.PCG64([seed, 31]))
    qd, kd = hp.nHead * hp.headDim, hp.nHeadKv * hp.headDim
    f = lambda *s: g.standard_normal(s, dtype=np.float32)  # noqa: E731
    m = Model(hp, f(hp.nLayer, hp.nVocab, qd), f(hp.nLayer, hp.nVocab, kd), f(hp.nLayer, hp.nVocab, kd),
              f(qd, hp.nVocab))
    if qk_norm:
        m.qNorm = g.uniform(0.9, 1.1, (hp.nLayer, hp.headDim)).astype(np.float32)
        m.kNorm = g.uniform(0.9, 1.1, (hp.nLayer, hp.headDim)).astype(np.float32)
    return m


@dataclass
class KvCache:
    """KvCache (src/hippo_leap/backend_types.nim:41-49): callers may reset ``curLen``."""
    c: KvCacheC = field(default_factory=KvCacheC)

    @property
    def curLen(self) -> int:
        return self.c.cur_len

    @curLen.setter
    def curLen(self, v: int):
        self.c.cur_len = v

    @property
    def maxLen(self) -> int:
        return self.c.max_len


def initKvCache(hp: HParams, maxLen: int, device: int = 0) -> KvCache:
    cache = KvCache()
    hpc = hp.c()
    _check(_lib().hl_backend_init_kv_cache(device, C.byref(hpc), maxLen, C.byref(cache.c)))
    return cache


def freeKvCache(cache: KvCache):
    _check(_lib().hl_backend_free_kv_cache(C.byref(cache.c)))


def loadModelBackend(m: Model, hp: HParams, device: int = 0):
    keep = [np.ascontiguousarray(a, np.float32) if a is not None else None
            for a in (m.eq, m.ek, m.ev, m.wout, m.qNorm, m.kNorm)]
    w = WeightsC(*[None if a is None else a.ctypes.data for a in keep])
    hpc = hp.c()
    _check(_lib().hl_backend_load_model(device, C.byref(hpc), C.byref(w)))


def unloadModelBackend():
    _check(_lib().hl_backend_unload_model())


def forwardPrefill(m: Model, tokens, cache: KvCache) -> np.ndarray:
    """Logits of the last prompt position, shape [1, nVocab]."""
    toks = np.ascontiguousarray(tokens, np.int32)
    logits = np.empty((1, m.hparams.nVocab), np.float32)
    _check(_lib().hl_backend_forward_prefill(toks.ctypes.data_as(C.POINTER(_i32)), toks.size, C.byref(cache.c),
                                             logits.ctypes.data_as(_f32p)))
    return logits


def forwardPrefillChunk(m: Model, tokens, cache: KvCache) -> np.ndarray:
    """Prefill continuing at position cache.curLen (chunked prompt, or a shared prefix kept in the cache); logits of the
    last token.  The reference has no such proc: its forwardPrefill restarts at position 0."""
    toks = np.ascontiguousarray(tokens, np.int32)
    logits = np.empty((1, m.hparams.nVocab), np.float32)
    _check(_lib().hl_backend_forward_prefill_chunk(toks.ctypes.data_as(C.POINTER(_i32)), toks.size, C.byref(cache.c),
                                                   logits.ctypes.data_as(_f32p)))
    return logits


def forwardDecode(m: Model, token: int, cache: KvCache) -> np.ndarray:
    logits = np.empty((1, m.hparams.nVocab), np.float32)
    _check(_lib().hl_backend_forward_decode(int(token), C.byref(cache.c), logits.ctypes.data_as(_f32p)))
    return logits


def forwardDecodeToken(m: Model, token: int, cache: KvCache) -> int:
    nxt = _i32()
    _check(_lib().hl_backend_forward_decode_token(int(token), C.byref(cache.c), C.byref(nxt)))
    return nxt.value


def forwardDecodeTokenTimed(m: Model, token: int, cache: KvCache):
    """Returns (next token, gpu milliseconds) -- the Nim proc writes gpuMs through a var."""
    nxt, ms = _i32(), C.c_float()
    _check(_lib().hl_backend_forward_decode_token_timed(int(token), C.byref(cache.c), C.byref(nxt), C.byref(ms)))
    return nxt.value, ms.value


def argmaxLast(logits: np.ndarray, nVocab: int) -> int:
    """First maximal index of the last position, both layouts (src/hippo_leap/sampling.nim:6-32)."""
    if logits.ndim != 2:
        raise ValueError("logits must be 2D")
    if logits.shape[0] == nVocab:
        return int(np.argmax(logits[:, -1]))
    if logits.shape[1] == nVocab:
        return int(np.argmax(logits[-1]))
    raise ValueError("logits shape mismatch for vocab")


def setDecodeGraph(enabled: bool):
    """forwardDecodeToken[Timed]: replay a captured CUDA graph per token (default) or launch kernel by kernel."""
    _check(_lib().hl_backend_set_decode_graph(int(enabled)))


def launchCount() -> int:
    return _lib().hl_backend_launch_count()


@dataclass
class GenerateResult:
    """GenerateResult of the reference (src/hippo_leap/inference.nim:17-23), token ids instead of text."""
    tokens: list
    promptTokens: int
    completionTokens: int
    totalTokens: int
    elapsedMs: float
    gpuMs: float


def generate(m, cache: KvCache, promptTokens, maxTokens: int, maxContextLen: int | None = None,
             stopTokenIds=(), procs=None) -> GenerateResult:
    """The reference's generate loop (src/hippo_leap/inference.nim:51-97) on token ids: reset curLen,
    one prefill, argmax, then forwardDecodeTokenTimed until maxTokens or a stop token.  ``procs`` is the module whose
    forwardPrefill / forwardDecodeTokenTimed are driven (this one by default, ``dense`` for the dense model)."""
    import time
    forwardPrefill = globals()["forwardPrefill"] if procs is None else procs.forwardPrefill
    forwardDecodeTokenTimed = globals()["forwardDecodeTokenTimed"] if procs is None else procs.forwardDecodeTokenTimed
    t0 = time.perf_counter()
    cache.curLen = 0
    prompt = list(promptTokens)
    if not prompt:
        return GenerateResult([], 0, 0, 0, 0.0, 0.0)
    max_ctx = cache.maxLen if maxContextLen is None else maxContextLen
    max_gen = min(maxTokens, max_ctx - len(prompt))
    if max_gen <= 0:
        return GenerateResult([], len(prompt), 0, len(prompt), 0.0, 0.0)
    nxt = argmaxLast(forwardPrefill(m, prompt, cache), m.hparams.nVocab)
    generated, gpu_ms = [nxt], 0.0
    for _ in range(1, max_gen):
        if nxt in stopTokenIds:
            break
        nxt, ms = forwardDecodeTokenTimed(m, nxt, cache)
        gpu_ms += ms
        generated.append(nxt)
    return GenerateResult(generated, len(prompt), len(generated), len(prompt) + len(generated),
                          (time.perf_counter() - t0) * 1e3, gpu_ms)
