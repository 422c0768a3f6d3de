"""Thin Python host layer over the C ABI: device buffers come from torch, compute from the .so.

Each method maps 1:1 to an entry point of ``include/hl_b200.h``; a non-zero status becomes a
``HlError`` (a ``ValueError``, the exception type the reference backends raise for bad shapes
and full caches, src/hippo_leap/backends/naive.nim:3969-3976, 4594-4599).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib as L


class HlError(ValueError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{L.STATUS_NAMES.get(code, code)}: {msg}")
        self.code = code


def theta_table(rope_dim: int, base: float) -> np.ndarray:
    """theta_i = powf(1/base, 2i/rope_dim) on the host (naive.nim:3850-3855)."""
    th = np.empty(rope_dim // 2, np.float32)
    rc = L.load().hl_b200_theta_table_h(base, rope_dim, th.ctypes.data_as(C.POINTER(C.c_float)))
    if rc != 0:
        raise HlError(rc, "theta_table: bad rope_dim or base")
    return th


def theta_llama3_scale(theta: np.ndarray, factor: float = 32.0, low_freq_factor: float = 1.0,
                       high_freq_factor: float = 4.0, original_ctx: int = 8192) -> np.ndarray:
    th = np.ascontiguousarray(theta, np.float32).copy()
    rc = L.load().hl_b200_theta_llama3_scale_h(th.ctypes.data_as(C.POINTER(C.c_float)), th.size,
                                               factor, low_freq_factor, high_freq_factor,
                                               original_ctx)
    if rc != 0:
        raise HlError(rc, "theta_llama3_scale: bad arguments")
    return th


@dataclass
class AttnShape:
    n_head: int
    n_head_kv: int
    head_dim: int
    rope_dim: int | None = None
    rope_mode: int = L.HL_ROPE_SPLIT_HALF
    rms_eps: float = 1e-6
    q_norm_w: torch.Tensor | None = None  # device float32 [head_dim]
    k_norm_w: torch.Tensor | None = None

    def c(self) -> L.AttnShapeC:
        for w in (self.q_norm_w, self.k_norm_w):
            if w is not None:
                assert w.is_cuda and w.dtype == torch.float32 and w.is_contiguous()
                assert w.numel() == self.head_dim
        return L.AttnShapeC(
            self.n_head, self.n_head_kv, self.head_dim,
            self.head_dim if self.rope_dim is None else self.rope_dim, self.rope_mode,
            self.rms_eps,
            None if self.q_norm_w is None else self.q_norm_w.data_ptr(),
            None if self.k_norm_w is None else self.k_norm_w.data_ptr())


def view_of(t: torch.Tensor) -> L.ViewC:
    """[n_tok, heads, head_dim] tensor (any strides, float32 or float16) -> hl_view."""
    assert t.is_cuda and t.dim() == 3, "expected a CUDA tensor shaped [n_tok, heads, head_dim]"
    if t.dtype == torch.float32:
        dt = L.HL_DTYPE_F32
    elif t.dtype == torch.float16:
        dt = L.HL_DTYPE_F16
    else:
        raise HlError(L.HL_ERR_ARG, f"dtype {t.dtype} is neither float32 nor float16")
    s = t.stride()
    return L.ViewC(t.data_ptr(), dt, s[0], s[1], s[2])


def _i32_dev(t: torch.Tensor) -> int:
    assert t.is_cuda and t.dtype == torch.int32 and t.is_contiguous()
    return t.data_ptr()


class KvPool:
    """Paged fp16 KV cache: per layer K and V pools [num_blocks, n_head_kv, block_tokens, hd]."""

    def __init__(self, ctx: "Context", handle, n_layers, n_head_kv, head_dim, block_tokens,
                 num_blocks):
        self.ctx, self.handle = ctx, handle
        self.n_layers, self.n_head_kv, self.head_dim = n_layers, n_head_kv, head_dim
        self.block_tokens, self.num_blocks = block_tokens, num_blocks

    def layer_ptrs(self, layer: int):
        k, v, n = C.c_void_p(), C.c_void_p(), C.c_size_t()
        rc = self.ctx.lib.hl_b200_kv_layer(self.handle, layer, C.byref(k), C.byref(v), C.byref(n))
        if rc != 0:
            raise HlError(rc, "kv_layer: bad layer")
        return k.value, v.value, n.value

    def destroy(self):
        if self.handle is not None and self.ctx.handle is not None:
            self.ctx.lib.hl_b200_kv_destroy(self.ctx.handle, self.handle)
        self.handle = None


class Context:
    """One per process and device (hl_ctx).  Not re-entrant."""

    def __init__(self, device: int = 0, stream: torch.cuda.Stream | None = None):
        self.lib = L.load()
        self.device = device
        h = C.c_void_p()
        rc = self.lib.hl_b200_create(device, None, C.byref(h))
        if rc != 0:
            raise HlError(rc, f"hl_b200_create(device={device}) failed: no usable sm_100 GPU "
                              "(this library has no CPU fallback)")
        self.handle = h
        self._stream = None
        if stream is not None:
            # torch's default stream has handle 0, which hl_b200_create reads as "make your
            # own stream"; set_stream adopts handle 0 as the legacy default stream.
            self.set_stream(stream)

    # -- plumbing ---------------------------------------------------------------------------
    def _check(self, rc: int):
        if rc != 0:
            raise HlError(rc, self.lib.hl_b200_last_error(self.handle).decode())

    def close(self):
        if self.handle is not None:
            self.lib.hl_b200_destroy(self.handle)
            self.handle = None

    def sync(self):
        self._check(self.lib.hl_b200_sync(self.handle))

    def set_stream(self, stream: torch.cuda.Stream):
        self._check(self.lib.hl_b200_set_stream(self.handle, C.c_void_p(stream.cuda_stream)))
        self._stream = stream

    def device_status(self):
        code, detail = C.c_int32(), C.c_int32()
        self._check(self.lib.hl_b200_device_status(self.handle, C.byref(code), C.byref(detail)))
        return code.value, detail.value

    def launch_count(self) -> int:
        return self.lib.hl_b200_launch_count(self.handle)

    def set_tuning(self, decode_chunk_tokens: int = 0, prefill_kernel: int = 0):
        self._check(self.lib.hl_b200_set_tuning(self.handle, decode_chunk_tokens, prefill_kernel))

    # -- rope / kv ---------------------------------------------------------------------------
    def set_rope(self, theta: np.ndarray):
        th = np.ascontiguousarray(theta, np.float32)
        self._check(self.lib.hl_b200_set_rope(self.handle, th.ctypes.data_as(C.POINTER(C.c_float)),
                                              th.size))

    def kv_create(self, n_layers, n_head_kv, head_dim, block_tokens, num_blocks, layer_n_head_kv=None) -> KvPool:
        """``layer_n_head_kv``: KV heads per layer (entries <= 0 take ``n_head_kv``), initGpuKvCache's layerNHeadKv."""
        h = C.c_void_p()
        if layer_n_head_kv is None:
            self._check(self.lib.hl_b200_kv_create(self.handle, n_layers, n_head_kv, head_dim,
                                                   block_tokens, num_blocks, C.byref(h)))
        else:
            assert len(layer_n_head_kv) == n_layers
            arr = (C.c_int32 * n_layers)(*[int(x) for x in layer_n_head_kv])
            self._check(self.lib.hl_b200_kv_create_layers(self.handle, n_layers, arr, n_head_kv, head_dim,
                                                          block_tokens, num_blocks, C.byref(h)))
        return KvPool(self, h, n_layers, n_head_kv, head_dim, block_tokens, num_blocks)

    def kv_append_seq(self, kv: KvPool, layer: int, shape: AttnShape, k, v, start_pos: int,
                      block_table: torch.Tensor):
        sc, kc, vc = shape.c(), view_of(k), view_of(v)
        self._check(self.lib.hl_b200_kv_append_seq(
            self.handle, kv.handle, layer, C.byref(sc), C.byref(kc), C.byref(vc), k.shape[0],
            start_pos, _i32_dev(block_table), block_table.numel()))

    def kv_append_batch(self, kv: KvPool, layer: int, shape: AttnShape, k, v,
                        ctx_lens: torch.Tensor, block_tables: torch.Tensor):
        sc, kc, vc = shape.c(), view_of(k), view_of(v)
        self._check(self.lib.hl_b200_kv_append_batch(
            self.handle, kv.handle, layer, C.byref(sc), C.byref(kc), C.byref(vc), k.shape[0],
            _i32_dev(ctx_lens), _i32_dev(block_tables), block_tables.shape[1]))

    # -- attention ---------------------------------------------------------------------------
    def attn_prefill(self, kv: KvPool, layer: int, shape: AttnShape, q, start_pos: int,
                     block_table: torch.Tensor, out: torch.Tensor | None = None,
                     timed: bool = False, gate: torch.Tensor | None = None):
        """``gate`` ([n_tok, n_head, hd] view): out <- sigmoid(gate) * out in the kernel epilogue."""
        if out is None:
            out = torch.empty((q.shape[0], shape.n_head, shape.head_dim), dtype=torch.float32,
                              device=q.device)
        sc, qc, oc = shape.c(), view_of(q), view_of(out)
        ms = C.c_float(0.0)
        if gate is None:
            self._check(self.lib.hl_b200_attn_prefill(
                self.handle, kv.handle, layer, C.byref(sc), C.byref(qc), q.shape[0], start_pos,
                _i32_dev(block_table), block_table.numel(), C.byref(oc),
                C.byref(ms) if timed else None))
        else:
            gc = view_of(gate)
            self._check(self.lib.hl_b200_attn_prefill_gated(
                self.handle, kv.handle, layer, C.byref(sc), C.byref(qc), q.shape[0], start_pos,
                _i32_dev(block_table), block_table.numel(), C.byref(gc), C.byref(oc),
                C.byref(ms) if timed else None))
        return (out, ms.value) if timed else out

    def attn_decode(self, kv: KvPool, layer: int, shape: AttnShape, q, ctx_lens: torch.Tensor,
                    max_ctx: int, block_tables: torch.Tensor, out: torch.Tensor | None = None,
                    timed: bool = False, gate: torch.Tensor | None = None):
        if out is None:
            out = torch.empty((q.shape[0], shape.n_head, shape.head_dim), dtype=torch.float32,
                              device=q.device)
        sc, qc, oc = shape.c(), view_of(q), view_of(out)
        ms = C.c_float(0.0)
        if gate is None:
            self._check(self.lib.hl_b200_attn_decode(
                self.handle, kv.handle, layer, C.byref(sc), C.byref(qc), q.shape[0],
                _i32_dev(ctx_lens), max_ctx, _i32_dev(block_tables), block_tables.shape[1],
                C.byref(oc), C.byref(ms) if timed else None))
        else:
            gc = view_of(gate)
            self._check(self.lib.hl_b200_attn_decode_gated(
                self.handle, kv.handle, layer, C.byref(sc), C.byref(qc), q.shape[0],
                _i32_dev(ctx_lens), max_ctx, _i32_dev(block_tables), block_tables.shape[1],
                C.byref(gc), C.byref(oc), C.byref(ms) if timed else None))
        return (out, ms.value) if timed else out

    # -- host-buffer forms (inputs and result in host memory; the call synchronises) ------------
    @staticmethod
    def _host_ptr(t: torch.Tensor):
        assert (not t.is_cuda) and t.dtype == torch.float32 and t.is_contiguous()
        return C.cast(t.data_ptr(), C.POINTER(C.c_float))

    def prefill_host(self, kv: KvPool, layer: int, shape: AttnShape, q_h, k_h, v_h, start_pos: int,
                     block_table: torch.Tensor, out_h: torch.Tensor, timed: bool = False):
        sc = shape.c()
        ms = C.c_float(0.0)
        self._check(self.lib.hl_b200_prefill_host(
            self.handle, kv.handle, layer, C.byref(sc), self._host_ptr(q_h), self._host_ptr(k_h),
            self._host_ptr(v_h), q_h.shape[0], start_pos, _i32_dev(block_table),
            block_table.numel(), self._host_ptr(out_h), C.byref(ms) if timed else None))
        return ms.value if timed else None

    def decode_step_host(self, kv: KvPool, layer: int, shape: AttnShape, q_h, k_h, v_h,
                         ctx_lens: torch.Tensor, max_ctx: int, block_tables: torch.Tensor,
                         out_h: torch.Tensor, timed: bool = False):
        sc = shape.c()
        ms = C.c_float(0.0)
        self._check(self.lib.hl_b200_decode_step_host(
            self.handle, kv.handle, layer, C.byref(sc), self._host_ptr(q_h), self._host_ptr(k_h),
            self._host_ptr(v_h), q_h.shape[0], _i32_dev(ctx_lens), max_ctx,
            _i32_dev(block_tables), block_tables.shape[1], self._host_ptr(out_h),
            C.byref(ms) if timed else None))
        return ms.value if timed else None

    def decode_step_host_call(self, kv: KvPool, layer: int, shape: AttnShape, q_h, k_h, v_h,
                              ctx_lens: torch.Tensor, max_ctx: int, block_tables: torch.Tensor, out_h: torch.Tensor):
        """The same call with its arguments marshalled once: returns a function of no arguments that makes the C call
        on the SAME buffers (a serving loop that refills fixed host buffers every step); raises like the method does."""
        sc = shape.c()
        args = (self.handle, kv.handle, layer, C.byref(sc), self._host_ptr(q_h), self._host_ptr(k_h), self._host_ptr(v_h),
                q_h.shape[0], _i32_dev(ctx_lens), max_ctx, _i32_dev(block_tables), block_tables.shape[1],
                self._host_ptr(out_h), None)
        fn, check, keep = self.lib.hl_b200_decode_step_host, self._check, (sc, q_h, k_h, v_h, ctx_lens, block_tables, out_h)

        def call():
            check(fn(*args))
            return keep[-1]
        return call

    def attn_decode_static(self, kv: KvPool, layer: int, shape: AttnShape, q, ctx_lens: torch.Tensor,
                           max_ctx: int, block_tables: torch.Tensor, out: torch.Tensor):
        """hl_b200_attn_decode_static: the decode step with no allocation inside the library.

        For serving loops that own all device memory or cannot stall on cudaMalloc: the split-KV
        scratch is a fixed array in the library (limit: batch * n_head * chunks <= 32768, else
        HlError/HL_ERR_CAPACITY).  ``out`` must be supplied by the caller.  Calls share the scratch:
        do not let two of them overlap on the GPU.  Make the first call per device at start-up.
        """
        sc, qc, oc = shape.c(), view_of(q), view_of(out)
        self._check(self.lib.hl_b200_attn_decode_static(
            self.handle, kv.handle, layer, C.byref(sc), C.byref(qc), q.shape[0], _i32_dev(ctx_lens),
            max_ctx, _i32_dev(block_tables), block_tables.shape[1], C.byref(oc)))
        return out

    def selftest_wait_timeout(self, max_polls: int = 1000):
        """Launch the bounded-wait self-test; read the outcome with ``device_status()``."""
        self._check(self.lib.hl_b200_selftest_wait_timeout(self.handle, max_polls))

    def attn_prefill_bcast(self, kv: KvPool, layer: int, shape: AttnShape, q, start_pos: int,
                           block_table: torch.Tensor, out: torch.Tensor, peer_ptrs, timed: bool = False):
        """hl_b200_attn_prefill_bcast: prefill whose epilogue also stores each tile to ``peer_ptrs``
        (device addresses of the same output slice on other GPUs)."""
        sc, qc, oc = shape.c(), view_of(q), view_of(out)
        arr = (C.c_void_p * max(1, len(peer_ptrs)))(*peer_ptrs)
        ms = C.c_float(0.0)
        self._check(self.lib.hl_b200_attn_prefill_bcast(
            self.handle, kv.handle, layer, C.byref(sc), C.byref(qc), q.shape[0], start_pos,
            _i32_dev(block_table), block_table.numel(), C.byref(oc), arr, len(peer_ptrs),
            C.byref(ms) if timed else None))
        return (out, ms.value) if timed else out

    def attn_decode_bcast(self, kv: KvPool, layer: int, shape: AttnShape, q, ctx_lens: torch.Tensor, max_ctx: int,
                          block_tables: torch.Tensor, out: torch.Tensor, peer_ptrs, timed: bool = False):
        """hl_b200_attn_decode_bcast: the decode step whose kernels also store each output row to ``peer_ptrs``
        (device addresses of the same output slice on other GPUs)."""
        sc, qc, oc = shape.c(), view_of(q), view_of(out)
        arr = (C.c_void_p * max(1, len(peer_ptrs)))(*peer_ptrs)
        ms = C.c_float(0.0)
        self._check(self.lib.hl_b200_attn_decode_bcast(
            self.handle, kv.handle, layer, C.byref(sc), C.byref(qc), q.shape[0], _i32_dev(ctx_lens), max_ctx,
            _i32_dev(block_tables), block_tables.shape[1], C.byref(oc), arr, len(peer_ptrs),
            C.byref(ms) if timed else None))
        return (out, ms.value) if timed else out

    def linear_f16(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                   resid: torch.Tensor | None = None, out_dtype=torch.float32, timed: bool = False):
        """out[M, N] = a[M, K] @ w[N, K].T (+ resid): fp16 inputs, fp32 accumulation (hl_b200_linear_f16)."""
        assert a.is_cuda and w.is_cuda and a.dtype == torch.float16 and w.dtype == torch.float16
        assert a.dim() == 2 and w.dim() == 2 and a.stride(1) == 1 and w.stride(1) == 1 and a.shape[1] == w.shape[1]
        M, K = a.shape
        N = w.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        assert out.stride(1) == 1 and out.shape == (M, N)
        if resid is not None:
            assert resid.dtype == torch.float32 and resid.stride(1) == 1 and resid.shape == (M, N)
        ms = C.c_float(0.0)
        self._check(self.lib.hl_b200_linear_f16(
            self.handle, a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
            L.HL_DTYPE_F32 if out.dtype == torch.float32 else L.HL_DTYPE_F16, out.stride(0),
            None if resid is None else resid.data_ptr(), 0 if resid is None else resid.stride(0), M, N, K,
            C.byref(ms) if timed else None))
        return (out, ms.value) if timed else out

    def linear_f16_silu(self, a: torch.Tensor, w_gate_up: torch.Tensor, h: torch.Tensor | None = None):
        """h[M, N/2] = fp16(silu(gate) * up) of the merged projection whose weight rows interleave gate and up
        (hl_b200_linear_f16_silu); M >= 16."""
        assert a.is_cuda and w_gate_up.is_cuda and a.dtype == torch.float16 and w_gate_up.dtype == torch.float16
        assert a.stride(1) == 1 and w_gate_up.stride(1) == 1 and a.shape[1] == w_gate_up.shape[1]
        M, K = a.shape
        N = w_gate_up.shape[0]
        if h is None:
            h = torch.empty((M, N // 2), dtype=torch.float16, device=a.device)
        assert h.dtype == torch.float16 and h.stride(1) == 1 and h.shape == (M, N // 2)
        self._check(self.lib.hl_b200_linear_f16_silu(self.handle, a.data_ptr(), a.stride(0), w_gate_up.data_ptr(),
                                                     w_gate_up.stride(0), h.data_ptr(), h.stride(0), M, N, K, None))
        return h
