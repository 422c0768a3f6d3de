// KV append: K <- (RMSNorm) -> RoPE -> fp16 (RN-even) -> paged store;  V <- fp16 -> paged store.
// Replaces qkNorm*(K), rope*(K), storeKV*, fusedRopeStoreKV of the reference
// (src/hippo_leap/backends/naive.nim:2887-2971, 3006-3086, 3149-3285).  K is rotated exactly once,
// when it enters the cache, as the reference does (naive.nim:4074-4076).
// Memory-bound and small: one warp per (token, kv-head) row.
#pragma once
#include "hl_device.cuh"

namespace hl {

struct AppendArgs {
  View k, v;
  __half* k_pool;
  __half* v_pool;
  const float* k_norm_w;
  const float* theta;
  const int32_t* ctx_lens;      // batch mode: token i is sequence i at position ctx_lens[i]-1
  const int32_t* block_tables;  // [n_seq][max_blocks]
  int32_t* status;
  float eps;
  int32_t n_tok, start_pos, batch_mode;
  int32_t n_head_kv, rope_dim, rope_mode;
  int32_t block_tokens, num_blocks, max_blocks;
};

template <int HD>
__global__ void __launch_bounds__(128) kv_append_kernel(AppendArgs a) {
  __shared__ float rows[4][HD];
  // With programmatic stream serialisation this grid first waits for the kernel in front, which produced the K / V rows
  // it reads -- and the query rows the attention kernel behind it reads in ITS prologue, so only now may that kernel
  // start (its set-up and query prologue then overlap this append; it waits for this grid before it touches the cache).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  if (row >= static_cast<int64_t>(a.n_tok) * a.n_head_kv) return;
  const int t = static_cast<int>(row / a.n_head_kv);
  const int h = static_cast<int>(row % a.n_head_kv);
  const int pos = a.batch_mode ? a.ctx_lens[t] - 1 : a.start_pos + t;
  const int seq = a.batch_mode ? t : 0;
  const int lb = pos / a.block_tokens;
  if (pos < 0 || lb >= a.max_blocks) {
    if (lane == 0) report(a.status, HL_ERR_CAPACITY, t);
    return;
  }
  const int pb = a.block_tables[static_cast<int64_t>(seq) * a.max_blocks + lb];
  if (pb < 0 || pb >= a.num_blocks) {
    if (lane == 0) report(a.status, HL_ERR_BOUNDS, t);
    return;
  }
  const int64_t dst =
      ((static_cast<int64_t>(pb) * a.n_head_kv + h) * a.block_tokens + pos % a.block_tokens) * HD;

  float* x = rows[warp];
#pragma unroll
  for (int d = lane; d < HD; d += 32) x[d] = view_load(a.k, t, h, d);
  __syncwarp();
  norm_rope_row<HD>(x, a.k_norm_w, a.eps, a.theta, a.rope_dim, a.rope_mode, pos, lane);
#pragma unroll
  for (int p = lane; p < HD / 2; p += 32) {
    reinterpret_cast<__half2*>(a.k_pool + dst)[p] = __floats2half2_rn(x[2 * p], x[2 * p + 1]);
  }
#pragma unroll
  for (int p = lane; p < HD / 2; p += 32) {
    const float v0 = view_load(a.v, t, h, 2 * p), v1 = view_load(a.v, t, h, 2 * p + 1);
    reinterpret_cast<__half2*>(a.v_pool + dst)[p] = __floats2half2_rn(v0, v1);
  }
}

}  // namespace hl
