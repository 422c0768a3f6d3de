"""B200-native (sm_100a) attention hot path for hippo_leap.

RoPE (+ optional per-head QK RMSNorm), KV-cache append into a paged fp16 cache, causal
grouped-query attention for prefill and split-KV single-token attention for decode, as
hand-written CUDA kernels behind a C ABI (``include/hl_b200.h`` -> ``libhl_b200.so``).
``runtime`` wraps the ABI 1:1; ``backend`` mirrors the reference's backend contract
(initKvCache / loadModelBackend / forwardPrefill / forwardDecode ...).
Importing the package does not load the shared library; the first compute call does, and
raises if it is missing.  There is no CPU fallback.
"""
from ._lib import (HL_DTYPE_F16, HL_DTYPE_F32, HL_ROPE_INTERLEAVED, HL_ROPE_SPLIT_HALF, LIB_PATH)
from .runtime import AttnShape, Context, HlError, KvPool, theta_llama3_scale, theta_table

__all__ = ["AttnShape", "Context", "HlError", "KvPool", "theta_table", "theta_llama3_scale",
           "HL_ROPE_INTERLEAVED", "HL_ROPE_SPLIT_HALF", "HL_DTYPE_F32", "HL_DTYPE_F16", "LIB_PATH"]
