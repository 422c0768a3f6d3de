"""The backend contract on a dense llama / qwen3 model (``hl_dense_*`` in ``include/hl_backend.h``): same
procs, same meaning as ``backend.py``, but the model is a whole dense transformer -- embedding, RMSNorm,
Q/K/V/O projections, SwiGLU FFN, vocabulary projection -- with the attention hot path in the middle.
Weights are synthetic fp16 arrays (no GGUF reader here)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib as L
from .backend import KvCache, KvCacheC, argmaxLast  # noqa: F401  (same cache struct, same argmax rule)


class DenseHParamsC(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_vocab", "n_emb", "n_layer", "n_ffn", "n_head", "n_head_kv", "head_dim",
                                         "rope_dim")] + [("rope_freq_base", C.c_float), ("rms_eps", C.c_float),
                                                         ("rope_mode", C.c_int32), ("llama3_scaling", C.c_int32)]


_W_FIELDS = ("tok_emb", "attn_norm", "wq", "wk", "wv", "wo", "q_norm", "k_norm", "ffn_norm", "w_gate", "w_up", "w_down",
             "out_norm", "w_out")


class DenseWeightsC(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in _W_FIELDS]


_f32p, _i32 = C.POINTER(C.c_float), C.c_int32
DENSE_SYMBOLS = {
    "hl_dense_init_kv_cache": (_i32, [_i32, C.POINTER(DenseHParamsC), _i32, C.POINTER(KvCacheC)]),
    "hl_dense_free_kv_cache": (_i32, [C.POINTER(KvCacheC)]),
    "hl_dense_load_model": (_i32, [_i32, C.POINTER(DenseHParamsC), C.POINTER(DenseWeightsC)]),
    "hl_dense_unload_model": (_i32, []),
    "hl_dense_forward_prefill": (_i32, [C.POINTER(_i32), _i32, C.POINTER(KvCacheC), _f32p]),
    "hl_dense_forward_prefill_chunk": (_i32, [C.POINTER(_i32), _i32, C.POINTER(KvCacheC), _f32p]),
    "hl_dense_forward_decode": (_i32, [_i32, C.POINTER(KvCacheC), _f32p]),
    "hl_dense_forward_decode_token_timed": (_i32, [_i32, C.POINTER(KvCacheC), C.POINTER(_i32), _f32p]),
    "hl_dense_batch_create": (_i32, [_i32, _i32, C.POINTER(C.c_void_p)]),
    "hl_dense_batch_destroy": (_i32, [C.c_void_p]),
    "hl_dense_batch_seq_len": (_i32, [C.c_void_p, _i32]),
    "hl_dense_batch_prefill": (_i32, [C.c_void_p, _i32, C.POINTER(_i32), _i32, _i32, _f32p]),
    "hl_dense_batch_decode": (_i32, [C.c_void_p, C.POINTER(_i32), C.POINTER(_i32), _i32, C.POINTER(_i32), _f32p, _f32p]),
    "hl_dense_set_decode_graph": (_i32, [_i32]),
    "hl_dense_last_error": (C.c_char_p, []),
}
_typed = False


def _lib():
    global _typed
    lib = L.load()
    if not _typed:
        for name, (res, args) in DENSE_SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _typed = True
    return lib


def _check(rc: int):
    if rc != 0:
        raise ValueError(f"{L.STATUS_NAMES.get(rc, rc)}: {_lib().hl_dense_last_error().decode()}")


@dataclass
class DenseHParams:
    nVocab: int
    nEmb: int
    nLayer: int
    nFfn: int
    nHead: int
    nHeadKv: int
    headDim: int
    ropeDim: int = 0
    ropeFreqBase: float = 10000.0
    rmsEps: float = 1e-5
    ropeMode: int = L.HL_ROPE_SPLIT_HALF
    llama3Scaling: bool = False

    def c(self) -> DenseHParamsC:
        return DenseHParamsC(self.nVocab, self.nEmb, self.nLayer, self.nFfn, self.nHead, self.nHeadKv, self.headDim,
                             self.ropeDim, self.ropeFreqBase, self.rmsEps, self.ropeMode, int(self.llama3Scaling))


@dataclass
class DenseModel:
    """hparams + host weights: fp16 matrices [out, in] per layer, float32 norm vectors."""
    hparams: DenseHParams
    w: dict


def random_dense_model(hp: DenseHParams, seed: int, qk_norm: bool = False) -> DenseModel:
    """Seeded weights scaled like a trained model's (1/sqrt(fan_in)), norm gains ~U(0.9, 1.1)."""
    g = np.random.Generator(np.random.PCG64([seed, 77]))
    L_, E, F, V, hd = hp.nLayer, hp.nEmb, hp.nFfn, hp.nVocab, hp.headDim
    qd, kd = hp.nHead * hd, hp.nHeadKv * hd

    def mat(*shape):
        return (g.standard_normal(shape, dtype=np.float32) / np.sqrt(shape[-1])).astype(np.float16)

    def gain(*shape):
        return g.uniform(0.9, 1.1, shape).astype(np.float32)

    w = dict(tok_emb=g.standard_normal((V, E), dtype=np.float32).astype(np.float16), attn_norm=gain(L_, E),
             wq=mat(L_, qd, E), wk=mat(L_, kd, E), wv=mat(L_, kd, E), wo=mat(L_, E, qd),
             q_norm=gain(L_, hd) if qk_norm else None, k_norm=gain(L_, hd) if qk_norm else None,
             ffn_norm=gain(L_, E), w_gate=mat(L_, F, E), w_up=mat(L_, F, E), w_down=mat(L_, E, F), out_norm=gain(E),
             w_out=mat(V, E))
    return DenseModel(hp, w)


def initKvCache(hp: DenseHParams, maxLen: int, device: int = 0) -> KvCache:
    cache = KvCache()
    hpc = hp.c()
    _check(_lib().hl_dense_init_kv_cache(device, C.byref(hpc), maxLen, C.byref(cache.c)))
    return cache


def freeKvCache(cache: KvCache):
    _check(_lib().hl_dense_free_kv_cache(C.byref(cache.c)))


def loadModelBackend(m: DenseModel, hp: DenseHParams, device: int = 0):
    keep = {k: (None if v is None else np.ascontiguousarray(v)) for k, v in m.w.items()}
    wc = DenseWeightsC(*[None if keep[n] is None else keep[n].ctypes.data for n in _W_FIELDS])
    hpc = hp.c()
    _check(_lib().hl_dense_load_model(device, C.byref(hpc), C.byref(wc)))


def unloadModelBackend():
    _check(_lib().hl_dense_unload_model())


def forwardPrefill(m: DenseModel, tokens, cache: KvCache) -> np.ndarray:
    toks = np.ascontiguousarray(tokens, np.int32)
    logits = np.empty((1, m.hparams.nVocab), np.float32)
    _check(_lib().hl_dense_forward_prefill(toks.ctypes.data_as(C.POINTER(_i32)), toks.size, C.byref(cache.c),
                                           logits.ctypes.data_as(_f32p)))
    return logits


def forwardPrefillChunk(m: DenseModel, tokens, cache: KvCache) -> np.ndarray:
    """Prefill continuing at position cache.curLen (chunked prompt, or a shared prefix kept in the cache)."""
    toks = np.ascontiguousarray(tokens, np.int32)
    logits = np.empty((1, m.hparams.nVocab), np.float32)
    _check(_lib().hl_dense_forward_prefill_chunk(toks.ctypes.data_as(C.POINTER(_i32)), toks.size, C.byref(cache.c),
                                                 logits.ctypes.data_as(_f32p)))
    return logits


def forwardDecode(m: DenseModel, token: int, cache: KvCache) -> np.ndarray:
    logits = np.empty((1, m.hparams.nVocab), np.float32)
    _check(_lib().hl_dense_forward_decode(int(token), C.byref(cache.c), logits.ctypes.data_as(_f32p)))
    return logits


def forwardDecodeTokenTimed(m: DenseModel, token: int, cache: KvCache):
    nxt, ms = _i32(), C.c_float()
    _check(_lib().hl_dense_forward_decode_token_timed(int(token), C.byref(cache.c), C.byref(nxt), C.byref(ms)))
    return nxt.value, ms.value


def setDecodeGraph(enabled: bool):
    _check(_lib().hl_dense_set_decode_graph(int(enabled)))


def forwardDecodeToken(m: DenseModel, token: int, cache: KvCache) -> int:
    return forwardDecodeTokenTimed(m, token, cache)[0]


class DecodeBatch:
    """Several sequences of the loaded model in one shared page pool, decoded together (hl_dense_batch_*): a
    continuous-batching hook.  The reference serves one sequence per process."""

    def __init__(self, m: DenseModel, max_seqs: int, max_len: int):
        self.n_vocab = m.hparams.nVocab
        self.handle = C.c_void_p()
        _check(_lib().hl_dense_batch_create(max_seqs, max_len, C.byref(self.handle)))

    def close(self):
        if self.handle:
            _lib().hl_dense_batch_destroy(self.handle)
            self.handle = C.c_void_p()

    def seq_len(self, seq: int) -> int:
        return _lib().hl_dense_batch_seq_len(self.handle, seq)

    def prefill(self, seq: int, tokens, start_pos: int = 0) -> np.ndarray:
        toks = np.ascontiguousarray(tokens, np.int32)
        logits = np.empty((1, self.n_vocab), np.float32)
        _check(_lib().hl_dense_batch_prefill(self.handle, seq, toks.ctypes.data_as(C.POINTER(_i32)), toks.size, start_pos,
                                             logits.ctypes.data_as(_f32p)))
        return logits

    def decode(self, seq_ids, tokens, want_logits: bool = False, timed: bool = False):
        """One step for the given sequences.  Returns (next_tokens [n], logits [n, nVocab] or None[, gpu ms])."""
        ids = np.ascontiguousarray(seq_ids, np.int32)
        toks = np.ascontiguousarray(tokens, np.int32)
        assert ids.shape == toks.shape and ids.ndim == 1
        nxt = np.empty(ids.size, np.int32)
        logits = np.empty((ids.size, self.n_vocab), np.float32) if want_logits else None
        ms = C.c_float(0.0)
        _check(_lib().hl_dense_batch_decode(self.handle, ids.ctypes.data_as(C.POINTER(_i32)), toks.ctypes.data_as(C.POINTER(_i32)),
                                            ids.size, nxt.ctypes.data_as(C.POINTER(_i32)),
                                            logits.ctypes.data_as(_f32p) if want_logits else None, C.byref(ms) if timed else None))
        return (nxt, logits, ms.value) if timed else (nxt, logits)
