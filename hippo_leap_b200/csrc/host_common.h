// Host-side objects behind the opaque handles of include/hl_b200.h.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <string>
#include <vector>

#include "../../include/hl_b200.h"

struct hl_ctx {
  int device = 0;
  int n_sm = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev2 = nullptr, ev3 = nullptr;
  float* theta_d = nullptr;  // RoPE theta table [theta_half]
  int theta_half = 0;
  int32_t* status_d = nullptr;  // {code, detail} written by bounded waits / bounds checks
  float* part_o = nullptr;      // split-KV partial outputs (grow-only scratch)
  float* part_ml = nullptr;     // split-KV partial (max, sum)
  size_t part_cap = 0;          // capacity in 128-float slots (one per (sequence, head, chunk); two at head_dim 256)
  // Set only by hl_b200_decode_step_host while it runs slices of one batch as concurrent chains: first slot of the
  // slice in the scratch (which it has sized for the whole batch beforehand), and the chunk length of the whole batch.
  size_t part_base = 0;
  int32_t chunk_override = 0;
  cudaStream_t side_stream[3] = {nullptr, nullptr, nullptr};
  cudaEvent_t side_done[3] = {nullptr, nullptr, nullptr};
  cudaEvent_t fork_ev = nullptr;
  // Bumped whenever one of the grow-only scratch buffers below is re-allocated: a captured CUDA graph that baked
  // the old address in must be captured again (the backends compare this before every replay).
  uint64_t scratch_epoch = 0;
  float* splitk_part = nullptr;   // split-K partial tiles of the several-row projections
  size_t splitk_cap = 0;          // in floats
  void* stage[4] = {nullptr, nullptr, nullptr, nullptr};  // q, k, v, out staging of the *_host calls
  size_t stage_cap[4] = {0, 0, 0, 0};
  void* cs_table = nullptr;  // float2 [cs_len][cs_half]: (cos, sin) of float(pos) * theta_i
  int cs_len = 0, cs_half = 0;
  void* encode_tiled = nullptr;  // cuTensorMapEncodeTiled, resolved through the runtime
  // Set by the backends inside this library (hl_backend_*, hl_dense_*), whose call order guarantees that the KV append
  // sits between the kernel that produced the query rows and the attention kernel: the attention kernels may then read
  // the query rows BEFORE griddepcontrol.wait (their prologue overlaps the append).  Through the public operators the
  // caller's kernel order is unknown -- the query rows may come from the kernel directly in front, and that kernel may
  // let its dependents start early -- so there every input is read after the wait.
  bool chain_pdl = false;
  int32_t decode_chunk = 0;
  int32_t prefill_kernel = 0;
  int64_t launches = 0;
  std::string err;
};

struct hl_kv {
  int n_layers = 0, n_head_kv = 0, head_dim = 0, block_tokens = 0, num_blocks = 0;
  size_t bytes_each = 0;                     // of a layer with n_head_kv KV heads
  std::vector<int> layer_kvh;                // KV heads of each layer (initGpuKvCache's layerNHeadKv, naive.nim:3562-3563)
  std::vector<size_t> layer_bytes;           // bytes of each layer's K (or V) pool
  std::vector<__half*> k, v;                 // per layer pools
  std::vector<CUtensorMap> k_map, v_map;     // 16-row x 64-column boxes, 128-byte swizzle
  std::vector<CUtensorMap> k_map128, v_map128;  // 128-row boxes when a block holds >= 128 tokens
};

int32_t hl_fail(hl_ctx* ctx, int32_t code, const char* fmt, ...);

// Argument checks shared by every attention entry point (defined in hl_b200.cu): the shape against the KV pool and
// the RoPE table; a view's pointer (non-null, aligned to its element size) and dtype.
int32_t hl_check_shape(hl_ctx* ctx, const hl_kv* kv, const hl_attn_shape* s, int32_t layer);
int32_t hl_check_view(hl_ctx* ctx, const hl_view* v, const char* name);
// Tokens per split-KV chunk of a decode launch: the tuning value, or about eight CTAs per SM within 128..1024.
int32_t hl_decode_chunk_tokens(const hl_ctx* ctx, int32_t batch, int32_t n_head_kv, int32_t max_ctx);
// Grows the split-KV partials scratch to `slots` 128-float slots (synchronises the context's stream if it must re-allocate).
int32_t hl_decode_reserve(hl_ctx* ctx, size_t slots);

// Decode projection (linear_gemv.cuh), 1 <= M <= 4.  mode 0: a = fp16 rows; mode 1: a = fp32 rows (lda in floats),
// RMSNorm with norm_w fused in front.  swiglu != 0: W rows interleave gate / up, out[M][N / 2] = fp16 silu(gate) * up.
int32_t hl_linear_decode_fused(hl_ctx* ctx, int32_t mode, int32_t swiglu, const void* a, int64_t lda, const float* norm_w,
                               float eps, const void* w, int64_t ldw, void* out, int32_t out_dtype, int64_t ldo,
                               const float* resid, int64_t ldr, int32_t M, int32_t N, int32_t K);

// Launch with programmatic stream serialisation: the grid may start while its predecessor in the stream drains; the
// kernels order themselves with griddepcontrol.wait.  HL_B200_NO_PDL in the environment restores plain launches.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args&&... args) {
  static const bool no_pdl = getenv("HL_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = no_pdl ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// The body of hl_b200_linear_f16 with the internal output forms; ld_store > 0 overrides the stored row stride.
int32_t hl_linear_f16_impl(hl_ctx* ctx, const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int32_t out_dtype,
                           int64_t ldo, const float* resid, int64_t ldr, int32_t M, int32_t N, int32_t K, float* gpu_ms,
                           int64_t ld_store = 0);

#define HL_CUDA(ctx, expr)                                                                   \
  do {                                                                                       \
    cudaError_t e_ = (expr);                                                                 \
    if (e_ != cudaSuccess)                                                                   \
      return hl_fail(ctx, HL_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                     __FILE__, __LINE__);                                                    \
  } while (0)
