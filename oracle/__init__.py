"""ctypes front of the CPU oracle (``tensor_ref.c``).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark import this
package; the product package never does.  Parity is unpinned by the reference's own tests
(see the header of ``tensor_ref.c``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

ROPE_INTERLEAVED = 0  # tensor.nim:156-166 pairs (2i, 2i+1)
ROPE_SPLIT_HALF = 1   # backends/naive.nim:3025-3030 pairs (i, i+half)


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with the Makefile beside this file."""
    src = os.path.join(_HERE, "tensor_ref.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        fp = C.POINTER(C.c_float)
        L.hl_ref_matmul.argtypes = [fp, fp, fp, C.c_int, C.c_int, C.c_int]
        L.hl_ref_rmsnorm.argtypes = [fp, fp, fp, C.c_long, C.c_int, C.c_float]
        L.hl_ref_softmax_last_dim.argtypes = [fp, fp, C.c_long, C.c_int]
        L.hl_ref_rope_inplace.argtypes = [fp, C.c_long, C.c_int, C.c_int, C.c_float, C.c_int]
        L.hl_ref_theta_table.argtypes = [fp, C.c_int, C.c_float]
        L.hl_ref_rope_row.argtypes = [fp, C.c_int, fp, C.c_int, C.c_int]
        L.hl_ref_round_fp16.argtypes = [C.c_float]
        L.hl_ref_round_fp16.restype = C.c_float
        L.hl_ref_attn_forward.argtypes = [
            fp, fp, fp, fp, fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
            fp, C.c_int, fp, fp, C.c_float, C.c_int, C.POINTER(C.c_int32), C.c_long, fp, fp,
            C.c_int]
        L.hl_ref_attn_forward.restype = C.c_int
        L.hl_ref_attn_gate.argtypes = [fp, fp, C.c_long]
        L.hl_ref_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))


def matmul(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.float32)
    lib().hl_ref_matmul(_p(a), _p(b), _p(c), m, k, n)
    return c


def rmsnorm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().hl_ref_rmsnorm(_p(x), _p(w), _p(out), x.size // x.shape[-1], x.shape[-1], eps)
    return out


def softmax_last_dim(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().hl_ref_softmax_last_dim(_p(x), _p(out), x.size // x.shape[-1], x.shape[-1])
    return out


def rope_inplace(x: np.ndarray, base: float, start_pos: int = 0) -> None:
    """tensor.nim ropeInplace on a contiguous float32 array of shape [..., seqLen, dim]."""
    assert x.dtype == np.float32 and x.flags.c_contiguous and x.ndim >= 2
    seq_len, dim = x.shape[-2], x.shape[-1]
    lib().hl_ref_rope_inplace(_p(x), x.size // (seq_len * dim), seq_len, dim, base, start_pos)


def theta_table(rope_dim: int, base: float) -> np.ndarray:
    th = np.empty(rope_dim // 2, np.float32)
    lib().hl_ref_theta_table(_p(th), rope_dim, base)
    return th


def rope_row(x: np.ndarray, rope_dim: int, theta: np.ndarray, pos: int, mode: int) -> None:
    assert x.dtype == np.float32 and x.flags.c_contiguous
    lib().hl_ref_rope_row(_p(x), rope_dim, _p(_f32(theta)), pos, mode)


def round_fp16(a) -> np.ndarray:
    """RN-even float32 -> fp16 -> float32 (numpy's astype does the same rounding)."""
    return _f32(a).astype(np.float16).astype(np.float32)


class SeqCache:
    """The oracle's own KV cache of ONE sequence: float32 [max_len, n_head_kv, hd]."""

    def __init__(self, max_len: int, n_head_kv: int, hd: int):
        self.k = np.zeros((max_len, n_head_kv, hd), np.float32)
        self.v = np.zeros((max_len, n_head_kv, hd), np.float32)
        self.cur_len = 0
        self.max_len = max_len


def attn_forward(q, k, v, cache: SeqCache, *, theta, rope_mode: int, rope_dim: int | None = None,
                 q_norm_w=None, k_norm_w=None, eps: float = 1e-6, kv_fp16: bool = False,
                 rows=None, n_threads: int = 0, return_q_rot: bool = False):
    """QK-norm -> RoPE -> append -> causal GQA for T new tokens of one sequence.

    q [T, n_head, hd], k/v [T, n_head_kv, hd] float32.  Returns out [T, n_head, hd], or
    [n_rows, hd] when ``rows`` ([n_rows, 2] of (t, head)) is given.  Advances cache.cur_len.
    """
    q, k, v = _f32(q), _f32(k), _f32(v)
    T, n_head, hd = q.shape
    n_head_kv = k.shape[1]
    theta = _f32(theta)
    if rope_dim is None:
        rope_dim = 2 * theta.shape[0]
    assert theta.shape[0] * 2 == rope_dim
    qw = None if q_norm_w is None else _f32(q_norm_w)
    kw = None if k_norm_w is None else _f32(k_norm_w)
    if rows is None:
        out = np.empty((T, n_head, hd), np.float32)
        rows_p, n_rows = None, 0
    else:
        rows = np.ascontiguousarray(rows, dtype=np.int32).reshape(-1, 2)
        out = np.empty((rows.shape[0], hd), np.float32)
        rows_p, n_rows = rows.ctypes.data_as(C.POINTER(C.c_int32)), rows.shape[0]
    q_rot = np.empty_like(q) if return_q_rot else None
    rc = lib().hl_ref_attn_forward(
        _p(q), _p(k), _p(v), _p(cache.k), _p(cache.v), cache.cur_len, cache.max_len, T, n_head,
        n_head_kv, hd, rope_dim, _p(theta), rope_mode, _p(qw), _p(kw), eps, int(kv_fp16),
        rows_p, n_rows, _p(out), _p(q_rot), n_threads)
    if rc != 0:
        raise ValueError(f"hl_ref_attn_forward rejected its arguments (rc={rc})")
    cache.cur_len += T
    return (out, q_rot) if return_q_rot else out


def attn_gate(out, gate) -> np.ndarray:
    """sigmoid(gate) * out, elementwise float32 (naive.nim:2287-2293)."""
    o = _f32(out).copy()
    g = _f32(gate)
    assert o.shape == g.shape
    lib().hl_ref_attn_gate(_p(o), _p(g), o.size)
    return o


def max_threads() -> int:
    return lib().hl_ref_max_threads()
