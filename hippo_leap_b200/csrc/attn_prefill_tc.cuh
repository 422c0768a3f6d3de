// tcgen05 / TMEM causal GQA prefill (placeholder while the warp-MMA kernel is brought up).
#pragma once
#include "attn_prefill_mma.cuh"
#include "host_common.h"

inline bool hl_prefill_tc_supported(const hl::PrefillArgs&, int) { return false; }
inline bool hl_prefill_tc_default(const hl::PrefillArgs&, int) { return false; }
inline int32_t hl_launch_prefill_tc(hl_ctx* ctx, hl_kv*, int32_t, const hl::PrefillArgs&, int) {
  return hl_fail(ctx, HL_ERR_UNSUPPORTED, "tcgen05 prefill kernel not built");
}
