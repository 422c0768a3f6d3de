"""ctypes binding of ``libhl_b200.so`` (the C ABI in ``include/hl_b200.h``).

There is no fallback of any kind: if the shared library is missing or does not load, importing
the compute entry points raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhl_b200.so")

HL_OK, HL_ERR_ARG, HL_ERR_CAPACITY, HL_ERR_ALIGN, HL_ERR_CUDA = 0, 1, 2, 3, 4
HL_ERR_TIMEOUT, HL_ERR_BOUNDS, HL_ERR_UNSUPPORTED = 5, 6, 7
STATUS_NAMES = {0: "HL_OK", 1: "HL_ERR_ARG", 2: "HL_ERR_CAPACITY", 3: "HL_ERR_ALIGN",
                4: "HL_ERR_CUDA", 5: "HL_ERR_TIMEOUT", 6: "HL_ERR_BOUNDS",
                7: "HL_ERR_UNSUPPORTED"}
HL_DTYPE_F32, HL_DTYPE_F16 = 0, 1
HL_ROPE_INTERLEAVED, HL_ROPE_SPLIT_HALF = 0, 1


class AttnShapeC(C.Structure):
    _fields_ = [("n_head", C.c_int32), ("n_head_kv", C.c_int32), ("head_dim", C.c_int32),
                ("rope_dim", C.c_int32), ("rope_mode", C.c_int32), ("rms_eps", C.c_float),
                ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p)]


class ViewC(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("tok_stride", C.c_int64),
                ("head_stride", C.c_int64), ("dim_stride", C.c_int64)]


# name -> (restype, argtypes); every symbol include/hl_b200.h declares.
_vp, _i32, _f32p = C.c_void_p, C.c_int32, C.POINTER(C.c_float)
_shape_p, _view_p = C.POINTER(AttnShapeC), C.POINTER(ViewC)
SYMBOLS = {
    "hl_b200_create": (_i32, [_i32, _vp, C.POINTER(_vp)]),
    "hl_b200_destroy": (_i32, [_vp]),
    "hl_b200_last_error": (C.c_char_p, [_vp]),
    "hl_b200_sync": (_i32, [_vp]),
    "hl_b200_set_stream": (_i32, [_vp, _vp]),
    "hl_b200_device_status": (_i32, [_vp, C.POINTER(_i32), C.POINTER(_i32)]),
    "hl_b200_launch_count": (C.c_int64, [_vp]),
    "hl_b200_theta_table_h": (_i32, [C.c_float, _i32, _f32p]),
    "hl_b200_theta_llama3_scale_h": (_i32, [_f32p, _i32, C.c_float, C.c_float, C.c_float, _i32]),
    "hl_b200_set_rope": (_i32, [_vp, _f32p, _i32]),
    "hl_b200_kv_create": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, C.POINTER(_vp)]),
    "hl_b200_kv_create_layers": (_i32, [_vp, _i32, C.POINTER(_i32), _i32, _i32, _i32, _i32, C.POINTER(_vp)]),
    "hl_b200_kv_destroy": (_i32, [_vp, _vp]),
    "hl_b200_kv_layer": (_i32, [_vp, _i32, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(C.c_size_t)]),
    "hl_b200_kv_append_seq": (_i32, [_vp, _vp, _i32, _shape_p, _view_p, _view_p, _i32, _i32, _vp, _i32]),
    "hl_b200_kv_append_batch": (_i32, [_vp, _vp, _i32, _shape_p, _view_p, _view_p, _i32, _vp, _vp, _i32]),
    "hl_b200_attn_prefill": (_i32, [_vp, _vp, _i32, _shape_p, _view_p, _i32, _i32, _vp, _i32, _view_p, _f32p]),
    "hl_b200_attn_prefill_bcast": (_i32, [_vp, _vp, _i32, _shape_p, _view_p, _i32, _i32, _vp, _i32, _view_p, C.POINTER(_vp), _i32, _f32p]),
    "hl_b200_attn_decode": (_i32, [_vp, _vp, _i32, _shape_p, _view_p, _i32, _vp, _i32, _vp, _i32, _view_p, _f32p]),
    "hl_b200_attn_decode_bcast": (_i32, [_vp, _vp, _i32, _shape_p, _view_p, _i32, _vp, _i32, _vp, _i32, _view_p, C.POINTER(_vp), _i32, _f32p]),
    "hl_b200_attn_prefill_gated": (_i32, [_vp, _vp, _i32, _shape_p, _view_p, _i32, _i32, _vp, _i32, _view_p, _view_p, _f32p]),
    "hl_b200_attn_decode_gated": (_i32, [_vp, _vp, _i32, _shape_p, _view_p, _i32, _vp, _i32, _vp, _i32, _view_p, _view_p, _f32p]),
    "hl_b200_attn_decode_static": (_i32, [_vp, _vp, _i32, _shape_p, _view_p, _i32, _vp, _i32, _vp, _i32, _view_p]),
    "hl_b200_prefill_host": (_i32, [_vp, _vp, _i32, _shape_p, _f32p, _f32p, _f32p, _i32, _i32, _vp, _i32, _f32p, _f32p]),
    "hl_b200_decode_step_host": (_i32, [_vp, _vp, _i32, _shape_p, _f32p, _f32p, _f32p, _i32, _vp, _i32, _vp, _i32, _f32p, _f32p]),
    "hl_b200_linear_f16": (_i32, [_vp, _vp, C.c_int64, _vp, C.c_int64, _vp, _i32, C.c_int64, _vp, C.c_int64, _i32, _i32, _i32, _f32p]),
    "hl_b200_linear_f16_silu": (_i32, [_vp, _vp, C.c_int64, _vp, C.c_int64, _vp, C.c_int64, _i32, _i32, _i32, _f32p]),
    "hl_b200_selftest_wait_timeout": (_i32, [_vp, _i32]),
    "hl_b200_set_tuning": (_i32, [_vp, _i32, _i32]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and type every entry point.  Raises if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m hippo_leap_b200.build` "
                "(nvcc, sm_100a).  hippo_leap_b200 has no CPU or library fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
