// The backend contract on a dense llama / qwen3 model: the whole layer stack of the reference's
// lkAttentionFfn layers (src/hippo_leap/backends/naive.nim:4054-4086 prefill, 4656-4771 decode) on the
// GPU.  Per layer:  RMSNorm -> merged Q|K|V projection -> [QK-norm -> RoPE -> KV append -> attention]
// -> output projection + residual -> RMSNorm -> merged gate|up projection -> SiLU*up -> down projection
// + residual;  then final norm, vocabulary projection, argmax.  The bracket is the attention hot path
// (libhl_b200 entry points); the projections are hl_b200_linear_f16; the rest are the row-wise kernels
// of dense_ops.cuh.  C ABI: include/hl_backend.h (hl_dense_*).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/hl_backend.h"
#include "dense_ops.cuh"
#include "host_common.h"

namespace {

struct Dense {
  hl_ctx* ctx = nullptr;
  int device = -1;
  bool loaded = false;
  hl_dense_hparams hp{};
  // weights on the device
  __half *tok_emb = nullptr, *wqkv = nullptr, *wo = nullptr, *wgu = nullptr, *wdown = nullptr, *wout = nullptr;
  float *attn_norm = nullptr, *ffn_norm = nullptr, *out_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
  // activations (capacity in tokens)
  int cap = 0;
  float *x = nullptr, *qkv = nullptr, *logits = nullptr;
  __half *xn = nullptr, *attn = nullptr, *gu = nullptr, *h = nullptr;
  int32_t *tokens_d = nullptr, *ctx_len_d = nullptr, *table_d = nullptr, *next_d = nullptr, *cand_i = nullptr;
  float* cand_v = nullptr;
  int table_len = 0;
  int32_t* pinned = nullptr;  // [0..1] device status, [2] next token, [4] token id of the step, [5] its context length
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  // one decode step captured as a CUDA graph, replayed per token (fed by pinned[4..5] through copy nodes)
  bool use_graph = true;
  cudaGraphExec_t graph = nullptr;
  void* graph_kv = nullptr;
  int graph_max_len = 0;
  uint64_t buf_epoch = 0;                        // bumped when the activation buffers are re-allocated
  uint64_t graph_buf_epoch = 0, graph_ctx_epoch = 0;  // what the captured graph was recorded against
  int64_t graph_kernels = 0;  // kernels inside one replay
  std::string err;
} d;

int32_t dfail(int32_t code, const char* msg) {
  d.err = msg;
  return code;
}
int32_t dfail_ctx(int32_t code, const char* call) {
  const char* inner = d.ctx ? hl_b200_last_error(d.ctx) : "";
  d.err = (inner && *inner) ? std::string(inner) : std::string(call) + " failed";
  return code;
}
#define D_CUDA(expr)                                                         \
  do {                                                                       \
    cudaError_t e_ = (expr);                                                 \
    if (e_ != cudaSuccess) return dfail(HL_ERR_CUDA, cudaGetErrorString(e_)); \
  } while (0)
#define D_TRY(expr)                                  \
  do {                                               \
    int32_t rc_ = (expr);                            \
    if (rc_ != HL_OK) return dfail_ctx(rc_, #expr);  \
  } while (0)
#define D_PASS(expr)              \
  do {                            \
    int32_t rc_ = (expr);         \
    if (rc_ != HL_OK) return rc_; \
  } while (0)

int32_t ensure_ctx(int device) {
  if (d.ctx) return device == d.device ? HL_OK : dfail(HL_ERR_ARG, "dense backend already bound to another device");
  int32_t rc = hl_b200_create(device, nullptr, &d.ctx);
  if (rc != HL_OK) return dfail(rc, "hl_b200_create failed: no usable sm_100 device (no CPU fallback exists)");
  d.device = device;
  // this backend always queues the KV append between the kernel that produces the query rows and the attention kernel:
  // the attention kernels may start their query prologue while the append runs
  d.ctx->chain_pdl = true;
  return HL_OK;
}

int32_t check_hp(const hl_dense_hparams* hp) {
  if (!hp) return dfail(HL_ERR_ARG, "null hparams");
  if (hp->n_vocab <= 0 || hp->n_emb <= 0 || hp->n_layer <= 0 || hp->n_ffn <= 0 || hp->n_head <= 0 || hp->n_head_kv <= 0)
    return dfail(HL_ERR_ARG, "non-positive hparam");
  if (hp->n_head % hp->n_head_kv != 0) return dfail(HL_ERR_ARG, "GQA requires head_count divisible by head_count_kv");
  if (hp->head_dim != 64 && hp->head_dim != 128 && hp->head_dim != 256)
    return dfail(HL_ERR_UNSUPPORTED, "head_dim must be 64, 128 or 256");
  if ((hp->n_emb & 7) || (hp->n_ffn & 7)) return dfail(HL_ERR_ALIGN, "n_emb and n_ffn must be multiples of 8");
  return HL_OK;
}

template <typename T>
bool upload(T** dst, const void* src, size_t n) {
  return cudaMalloc(dst, n * sizeof(T)) == cudaSuccess && cudaMemcpy(*dst, src, n * sizeof(T), cudaMemcpyHostToDevice) == cudaSuccess;
}

int32_t ensure_act(int n) {
  if (n <= d.cap) return HL_OK;
  cudaStreamSynchronize(d.ctx->stream);
  for (float** p : {&d.x, &d.qkv}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  for (__half** p : {&d.xn, &d.attn, &d.gu, &d.h}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  if (d.tokens_d) cudaFree(d.tokens_d);
  d.tokens_d = nullptr;
  d.cap = 0;
  d.buf_epoch++;
  const size_t E = d.hp.n_emb, F = d.hp.n_ffn, qd = static_cast<size_t>(d.hp.n_head) * d.hp.head_dim,
               kd = static_cast<size_t>(d.hp.n_head_kv) * d.hp.head_dim, N = n;
  D_CUDA(cudaMalloc(&d.x, N * E * sizeof(float)));
  D_CUDA(cudaMalloc(&d.qkv, N * (qd + 2 * kd) * sizeof(float)));
  D_CUDA(cudaMalloc(&d.xn, N * E * sizeof(__half)));
  D_CUDA(cudaMalloc(&d.attn, N * qd * sizeof(__half)));
  D_CUDA(cudaMalloc(&d.gu, N * 2 * F * sizeof(__half)));
  D_CUDA(cudaMalloc(&d.h, N * F * sizeof(__half)));
  D_CUDA(cudaMalloc(&d.tokens_d, N * sizeof(int32_t)));
  d.cap = n;
  return HL_OK;
}

__global__ void set_i32(int32_t* p, int32_t v) { *p = v; }

// argmax over the vocabulary, first maximal index wins (src/hippo_leap/sampling.nim:13-19), in two launches:
// kArgmaxBlocks blocks each reduce a contiguous range to one (value, index) candidate, one block reduces those.
constexpr int kArgmaxBlocks = 128;

__device__ __forceinline__ void argmax_take(float& best, int& idx, float v, int i) {
  if (v > best || (v == best && i < idx)) {
    best = v;
    idx = i;
  }
}

__device__ __forceinline__ void argmax_block_reduce(float& best, int& idx) {
  __shared__ float bv[8];
  __shared__ int bi[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    argmax_take(best, idx, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) {
    bv[threadIdx.x >> 5] = best;
    bi[threadIdx.x >> 5] = idx;
  }
  __syncthreads();
  if (threadIdx.x == 0)
    for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) argmax_take(best, idx, bv[w], bi[w]);
}

// blockIdx.y: the row of logits (one per sequence of a batched step)
__global__ void __launch_bounds__(256) argmax_partial(const float* __restrict__ logits, int n, float* __restrict__ cand_v,
                                                      int32_t* __restrict__ cand_i) {
  logits += static_cast<int64_t>(blockIdx.y) * n;
  cand_v += blockIdx.y * kArgmaxBlocks;
  cand_i += blockIdx.y * kArgmaxBlocks;
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int beg = blockIdx.x * per, end = min(n, beg + per);
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = beg + threadIdx.x; i < end; i += 256) argmax_take(best, idx, logits[i], i);
  argmax_block_reduce(best, idx);
  if (threadIdx.x == 0) {
    cand_v[blockIdx.x] = best;
    cand_i[blockIdx.x] = idx;
  }
}

__global__ void __launch_bounds__(kArgmaxBlocks) argmax_final(const float* __restrict__ cand_v,
                                                              const int32_t* __restrict__ cand_i, int32_t* __restrict__ out) {
  float best = cand_v[blockIdx.x * kArgmaxBlocks + threadIdx.x];
  int idx = cand_i[blockIdx.x * kArgmaxBlocks + threadIdx.x];
  argmax_block_reduce(best, idx);
  if (threadIdx.x == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
}

void launch_argmax(cudaStream_t st);

// One forward over n tokens starting at position pos0; decode is n == 1.  `grid_ctx` sizes the decode grid and its
// scratch (>= the real context); with `from_pinned` the token id and the context length come from the pinned step
// record through copy nodes, so that a captured graph of the sequence can be replayed for every token.
//
// `bd` switches to a decode step over n DIFFERENT sequences of a shared pool (continuous batching): row i is one new
// token of the sequence whose context length (after the append) is bd->ctx_lens_d[i] and whose pages are row i of
// bd->tables_d; logits of all n rows go to bd->logits_d.
struct BatchDecode {
  hl_kv* kv;
  const int32_t* ctx_lens_d;  // [n]
  const int32_t* tables_d;    // [n][table_len]
  int table_len, max_ctx;
  float* logits_d;            // [n][n_vocab]
};
struct KvRef {
  hl_kv* kv;
  const int32_t* table;  // block table of the one sequence (prefill / single-sequence decode)
  int table_len;
};

// The identity block table is shared by all caches and only ever grows; each cache uses its own number of blocks
// as the table length, so a smaller cache created later does not shorten an older cache's view of it.
KvRef ref_of(const hl_kv_cache* cache) {
  hl_kv* kv = static_cast<hl_kv*>(cache->gpu_cache);
  return KvRef{kv, d.table_d, kv->num_blocks};
}

int32_t forward(const int32_t* tokens_h, int n, int pos0, KvRef ref, bool decode, int grid_ctx = 0,
                bool from_pinned = false, const BatchDecode* bd = nullptr) {
  using namespace hl;
  hl_kv* kv = bd ? bd->kv : ref.kv;
  const hl_dense_hparams& hp = d.hp;
  const int E = hp.n_emb, F = hp.n_ffn, hd = hp.head_dim, qd = hp.n_head * hd, kd = hp.n_head_kv * hd, qkvd = qd + 2 * kd;
  D_CUDA(cudaSetDevice(d.device));
  D_PASS(ensure_act(n));
  cudaStream_t st = d.ctx->stream;
  if (from_pinned) {
    D_CUDA(cudaMemcpyAsync(d.tokens_d, &d.pinned[4], sizeof(int32_t), cudaMemcpyHostToDevice, st));
    D_CUDA(cudaMemcpyAsync(d.ctx_len_d, &d.pinned[5], sizeof(int32_t), cudaMemcpyHostToDevice, st));
  } else {
    D_CUDA(cudaMemcpyAsync(d.tokens_d, tokens_h, n * sizeof(int32_t), cudaMemcpyHostToDevice, st));
    if (decode && !bd) set_i32<<<1, 1, 0, st>>>(d.ctx_len_d, pos0 + 1);
  }
  if (grid_ctx < pos0 + 1) grid_ctx = pos0 + 1;
  // one row: RMSNorm and SwiGLU run as prologue / epilogue of the GEMV next to them; more rows go through the row
  // kernels and the tcgen05 projections
  const bool fused = n == 1;
  embedding_f16_kernel<<<n, 128, 0, st>>>(d.tok_emb, d.tokens_d, E, hp.n_vocab, d.x);
  d.ctx->launches += 2;
  for (int l = 0; l < hp.n_layer; ++l) {
    hl_attn_shape s{};
    s.n_head = hp.n_head;
    s.n_head_kv = hp.n_head_kv;
    s.head_dim = hd;
    s.rope_dim = hp.rope_dim > 0 ? hp.rope_dim : hd;
    s.rope_mode = hp.rope_mode;
    s.rms_eps = hp.rms_eps;
    s.q_norm_w = d.q_norm ? d.q_norm + static_cast<size_t>(l) * hd : nullptr;
    s.k_norm_w = d.k_norm ? d.k_norm + static_cast<size_t>(l) * hd : nullptr;
    if (fused) {
      D_TRY(hl_linear_decode_fused(d.ctx, 1, 0, d.x, E, d.attn_norm + static_cast<size_t>(l) * E, hp.rms_eps,
                                   d.wqkv + static_cast<size_t>(l) * qkvd * E, E, d.qkv, HL_DTYPE_F32, qkvd, nullptr, 0, n,
                                   qkvd, E));
    } else {
      rmsnorm_rows_kernel<<<n, 256, 0, st>>>(d.x, d.attn_norm + static_cast<size_t>(l) * E, E, hp.rms_eps, d.xn);
      d.ctx->launches += 1;
      D_TRY(hl_b200_linear_f16(d.ctx, d.xn, E, d.wqkv + static_cast<size_t>(l) * qkvd * E, E, d.qkv, HL_DTYPE_F32, qkvd,
                               nullptr, 0, n, qkvd, E, nullptr));
    }
    hl_view qv{d.qkv, HL_DTYPE_F32, qkvd, hd, 1}, kvw{d.qkv + qd, HL_DTYPE_F32, qkvd, hd, 1},
        vv{d.qkv + qd + kd, HL_DTYPE_F32, qkvd, hd, 1}, ov{d.attn, HL_DTYPE_F16, qd, hd, 1};
    if (bd) {
      D_TRY(hl_b200_kv_append_batch(d.ctx, kv, l, &s, &kvw, &vv, n, bd->ctx_lens_d, bd->tables_d, bd->table_len));
      D_TRY(hl_b200_attn_decode(d.ctx, kv, l, &s, &qv, n, bd->ctx_lens_d, bd->max_ctx, bd->tables_d, bd->table_len, &ov,
                                nullptr));
    } else if (decode) {
      D_TRY(hl_b200_kv_append_batch(d.ctx, kv, l, &s, &kvw, &vv, 1, d.ctx_len_d, ref.table, ref.table_len));
      D_TRY(hl_b200_attn_decode(d.ctx, kv, l, &s, &qv, 1, d.ctx_len_d, grid_ctx, ref.table, ref.table_len, &ov, nullptr));
    } else {
      D_TRY(hl_b200_kv_append_seq(d.ctx, kv, l, &s, &kvw, &vv, n, pos0, ref.table, ref.table_len));
      D_TRY(hl_b200_attn_prefill(d.ctx, kv, l, &s, &qv, n, pos0, ref.table, ref.table_len, &ov, nullptr));
    }
    // x += attn . Wo^T   (output projection + residual, naive.nim:4079-4080)
    D_TRY(hl_b200_linear_f16(d.ctx, d.attn, qd, d.wo + static_cast<size_t>(l) * E * qd, qd, d.x, HL_DTYPE_F32, E, d.x, E, n,
                             E, qd, nullptr));
    if (fused) {
      // h = silu(gate) * up in the epilogue of the merged projection; x += h . Wdown^T   (naive.nim:4083-4086)
      D_TRY(hl_linear_decode_fused(d.ctx, 1, 1, d.x, E, d.ffn_norm + static_cast<size_t>(l) * E, hp.rms_eps,
                                   d.wgu + static_cast<size_t>(l) * 2 * F * E, E, d.h, HL_DTYPE_F16, F, nullptr, 0, n, 2 * F, E));
      D_TRY(hl_linear_decode_fused(d.ctx, 0, 0, d.h, F, nullptr, 0.f, d.wdown + static_cast<size_t>(l) * E * F, F, d.x,
                                   HL_DTYPE_F32, E, d.x, E, n, E, F));
    } else {
      rmsnorm_rows_kernel<<<n, 256, 0, st>>>(d.x, d.ffn_norm + static_cast<size_t>(l) * E, E, hp.rms_eps, d.xn);
      static const bool no_fused_silu = getenv("HL_B200_NO_FUSED_SILU") != nullptr;  // for comparison runs
      if (n > 128 && !no_fused_silu) {
        // SiLU(gate) * up in the GEMM's epilogue: no fp16 [n, 2F] intermediate, no row kernel.  (Up to 128 rows the
        // several-row projection kernel is the faster GEMM and keeps the two-step form.)
        D_TRY(hl_b200_linear_f16_silu(d.ctx, d.xn, E, d.wgu + static_cast<size_t>(l) * 2 * F * E, E, d.h, F, n, 2 * F, E,
                                      nullptr));
        d.ctx->launches -= 1;
      } else {
        D_TRY(hl_b200_linear_f16(d.ctx, d.xn, E, d.wgu + static_cast<size_t>(l) * 2 * F * E, E, d.gu, HL_DTYPE_F16, 2 * F,
                                 nullptr, 0, n, 2 * F, E, nullptr));
        const int64_t total = static_cast<int64_t>(n) * F;
        if ((total & 7) == 0 && ((reinterpret_cast<uintptr_t>(d.gu) | reinterpret_cast<uintptr_t>(d.h)) & 15) == 0) {
          const int64_t total8 = total >> 3;
          const int64_t want = (total8 + 255) / 256, cap = static_cast<int64_t>(d.ctx->n_sm) * 16;
          silu_mul_vec8_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, st>>>(d.gu, total8, d.h);
        } else {
          silu_mul_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(d.gu, F, total, d.h);
        }
      }
      d.ctx->launches += 2;
      // x += h . Wdown^T   (naive.nim:4085-4086)
      D_TRY(hl_b200_linear_f16(d.ctx, d.h, F, d.wdown + static_cast<size_t>(l) * E * F, F, d.x, HL_DTYPE_F32, E, d.x, E, n, E,
                               F, nullptr));
    }
  }
  if (bd) {
    // final norm + vocabulary projection of every row (each is the last position of its sequence)
    if (fused) {
      D_TRY(hl_linear_decode_fused(d.ctx, 1, 0, d.x, E, d.out_norm, hp.rms_eps, d.wout, E, bd->logits_d, HL_DTYPE_F32,
                                   hp.n_vocab, nullptr, 0, n, hp.n_vocab, E));
    } else {
      rmsnorm_rows_kernel<<<n, 256, 0, st>>>(d.x, d.out_norm, E, hp.rms_eps, d.xn);
      d.ctx->launches += 1;
      D_TRY(hl_b200_linear_f16(d.ctx, d.xn, E, d.wout, E, bd->logits_d, HL_DTYPE_F32, hp.n_vocab, nullptr, 0, n, hp.n_vocab,
                               E, nullptr));
    }
    D_CUDA(cudaGetLastError());
    return HL_OK;
  }
  // final norm + vocabulary projection of the LAST position only
  D_TRY(hl_linear_decode_fused(d.ctx, 1, 0, d.x + static_cast<size_t>(n - 1) * E, E, d.out_norm, hp.rms_eps, d.wout, E, d.logits,
                               HL_DTYPE_F32, hp.n_vocab, nullptr, 0, 1, hp.n_vocab, E));
  D_CUDA(cudaGetLastError());
  return HL_OK;
}

void launch_argmax(cudaStream_t st) {
  argmax_partial<<<kArgmaxBlocks, 256, 0, st>>>(d.logits, d.hp.n_vocab, d.cand_v, d.cand_i);
  argmax_final<<<1, kArgmaxBlocks, 0, st>>>(d.cand_v, d.cand_i, d.next_d);
  d.ctx->launches += 2;
}

int32_t finish() {
  D_CUDA(cudaMemcpyAsync(d.pinned, d.ctx->status_d, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, d.ctx->stream));
  D_CUDA(cudaStreamSynchronize(d.ctx->stream));
  if (d.pinned[0] != 0) {
    const int32_t code = d.pinned[0];
    cudaMemset(d.ctx->status_d, 0, 2 * sizeof(int32_t));
    return dfail(code, "a device-side check failed during the forward pass");
  }
  return HL_OK;
}

int32_t check_cache(const hl_kv_cache* cache) {
  if (!d.loaded) return dfail(HL_ERR_ARG, "no model loaded (loadModelBackend)");
  if (!cache || !cache->gpu_cache) return dfail(HL_ERR_ARG, "null KV cache (initKvCache)");
  return HL_OK;
}

// Capture one decode step (every layer, logits, argmax, result and status copies) into a CUDA graph.  The decode grid
// and the split-KV scratch are sized for the cache's capacity, so one graph serves every position.
int32_t ensure_decode_graph(hl_kv_cache* cache) {
  // still valid: same cache, and no buffer whose address the graph holds has been re-allocated since
  if (d.graph && d.graph_kv == cache->gpu_cache && d.graph_max_len == cache->max_len && d.graph_buf_epoch == d.buf_epoch &&
      d.graph_ctx_epoch == d.ctx->scratch_epoch)
    return HL_OK;
  if (d.graph) cudaGraphExecDestroy(d.graph);
  d.graph = nullptr;
  cudaStream_t st = d.ctx->stream;
  // an uncaptured pass first: it configures kernels and grows every scratch buffer, so nothing allocates or
  // synchronises during capture; the first replay repeats it at the same position with the same values
  D_PASS(forward(nullptr, 1, d.pinned[5] - 1, ref_of(cache), true, cache->max_len, true));
  D_CUDA(cudaStreamSynchronize(st));
  D_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
  const int64_t counted = d.ctx->launches;
  int32_t rc = forward(nullptr, 1, d.pinned[5] - 1, ref_of(cache), true, cache->max_len, true);
  if (rc == HL_OK) {
    launch_argmax(st);
    cudaMemcpyAsync(&d.pinned[2], d.next_d, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
    cudaMemcpyAsync(d.pinned, d.ctx->status_d, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  }
  d.graph_kernels = d.ctx->launches - counted;
  d.ctx->launches = counted;  // recorded, not launched
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(st, &graph);
  if (rc != HL_OK) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (e != cudaSuccess || !graph) return dfail(HL_ERR_CUDA, "stream capture of the decode step failed");
  e = cudaGraphInstantiate(&d.graph, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return dfail(HL_ERR_CUDA, "cudaGraphInstantiate failed");
  d.graph_kv = cache->gpu_cache;
  d.graph_max_len = cache->max_len;
  d.graph_buf_epoch = d.buf_epoch;
  d.graph_ctx_epoch = d.ctx->scratch_epoch;
  return HL_OK;
}

// One decode step by graph replay; logits_h (optional) receives the logits, next_token (optional) the argmax.
int32_t decode_graph(int32_t token, hl_kv_cache* cache, float* logits_h, int32_t* next_token, float* gpu_ms) {
  if (cache->cur_len < 0) return dfail(HL_ERR_ARG, "negative cur_len");
  D_CUDA(cudaSetDevice(d.device));
  d.pinned[4] = token;
  d.pinned[5] = cache->cur_len + 1;
  D_PASS(ensure_decode_graph(cache));
  cudaStream_t st = d.ctx->stream;
  const int64_t before = d.ctx->launches;
  if (gpu_ms) D_CUDA(cudaEventRecord(d.e0, st));
  D_CUDA(cudaGraphLaunch(d.graph, st));
  if (gpu_ms) D_CUDA(cudaEventRecord(d.e1, st));
  if (logits_h) D_CUDA(cudaMemcpyAsync(logits_h, d.logits, d.hp.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, st));
  D_CUDA(cudaStreamSynchronize(st));
  d.ctx->launches = before + d.graph_kernels;
  if (d.pinned[0] != 0) {
    const int32_t code = d.pinned[0];
    cudaMemset(d.ctx->status_d, 0, 2 * sizeof(int32_t));
    return dfail(code, "a device-side check failed during the decode step");
  }
  if (gpu_ms) D_CUDA(cudaEventElapsedTime(gpu_ms, d.e0, d.e1));
  if (next_token) *next_token = d.pinned[2];
  cache->cur_len += 1;
  return HL_OK;
}

}  // namespace

// ---- several sequences in one shared page pool, decoded together (continuous batching hook) ----------------------
struct hl_dense_batch {
  hl_kv* kv = nullptr;
  int max_seqs = 0, max_len = 0, nb = 0;
  std::vector<int32_t> cur_len;        // tokens held per sequence
  int32_t* tables_d = nullptr;         // [max_seqs][nb]: sequence s owns pages [s * nb, (s + 1) * nb)
  int32_t* act_tables_d = nullptr;     // [max_seqs][nb]: rows of the sequences of the current step
  int32_t* ctx_lens_d = nullptr;       // [max_seqs]
  int32_t *next_d = nullptr, *cand_i = nullptr;
  float *cand_v = nullptr, *logits_d = nullptr;  // [max_seqs][n_vocab]
  int32_t* pinned = nullptr;           // [0..1] status, then per step: next tokens [S], context lengths [S], token ids [S], tables [S][nb]
  std::vector<cudaGraphExec_t> graphs; // one captured decode step per number of active sequences (index n)
  std::vector<uint64_t> graph_epoch;   // buffer epochs (activations + library scratch) each was recorded against
};

extern "C" int32_t hl_dense_batch_create(int32_t max_seqs, int32_t max_len, hl_dense_batch** out) {
  if (!out) return dfail(HL_ERR_ARG, "null out");
  *out = nullptr;
  if (!d.loaded) return dfail(HL_ERR_ARG, "no model loaded (loadModelBackend)");
  if (max_seqs <= 0 || max_seqs > 4096 || max_len <= 0) return dfail(HL_ERR_ARG, "max_seqs must be 1..4096 and max_len positive");
  D_CUDA(cudaSetDevice(d.device));
  hl_dense_batch* b = new hl_dense_batch();
  b->max_seqs = max_seqs;
  b->max_len = max_len;
  b->nb = (max_len + 127) / 128;
  b->cur_len.assign(max_seqs, 0);
  b->graphs.assign(max_seqs + 1, nullptr);
  b->graph_epoch.assign(max_seqs + 1, 0);
  const size_t nt = static_cast<size_t>(max_seqs) * b->nb, V = d.hp.n_vocab;
  int32_t rc = hl_b200_kv_create(d.ctx, d.hp.n_layer, d.hp.n_head_kv, d.hp.head_dim, 128, static_cast<int32_t>(nt), &b->kv);
  std::vector<int32_t> ident(nt);
  for (size_t i = 0; i < nt; ++i) ident[i] = static_cast<int32_t>(i);
  const bool ok = rc == HL_OK && cudaMalloc(&b->tables_d, nt * 4) == cudaSuccess &&
                  cudaMemcpy(b->tables_d, ident.data(), nt * 4, cudaMemcpyHostToDevice) == cudaSuccess &&
                  cudaMalloc(&b->act_tables_d, nt * 4) == cudaSuccess && cudaMalloc(&b->ctx_lens_d, max_seqs * 4) == cudaSuccess &&
                  cudaMalloc(&b->next_d, max_seqs * 4) == cudaSuccess &&
                  cudaMalloc(&b->cand_i, static_cast<size_t>(max_seqs) * kArgmaxBlocks * 4) == cudaSuccess &&
                  cudaMalloc(&b->cand_v, static_cast<size_t>(max_seqs) * kArgmaxBlocks * 4) == cudaSuccess &&
                  cudaMalloc(&b->logits_d, static_cast<size_t>(max_seqs) * V * 4) == cudaSuccess &&
                  cudaMallocHost(&b->pinned, (2 + 3 * static_cast<size_t>(max_seqs) + nt) * 4) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    hl_dense_batch_destroy(b);
    return rc != HL_OK ? dfail_ctx(rc, "hl_b200_kv_create") : dfail(HL_ERR_CUDA, "allocation of the batch state failed");
  }
  *out = b;
  return HL_OK;
}

extern "C" int32_t hl_dense_batch_destroy(hl_dense_batch* b) {
  if (!b) return HL_OK;
  if (d.ctx) {
    cudaSetDevice(d.device);
    cudaStreamSynchronize(d.ctx->stream);
    if (b->kv) hl_b200_kv_destroy(d.ctx, b->kv);
  }
  for (int32_t** p : {&b->tables_d, &b->act_tables_d, &b->ctx_lens_d, &b->next_d, &b->cand_i})
    if (*p) cudaFree(*p);
  for (float** p : {&b->cand_v, &b->logits_d})
    if (*p) cudaFree(*p);
  for (cudaGraphExec_t ge : b->graphs)
    if (ge) cudaGraphExecDestroy(ge);
  if (b->pinned) cudaFreeHost(b->pinned);
  delete b;
  return HL_OK;
}

extern "C" int32_t hl_dense_batch_seq_len(const hl_dense_batch* b, int32_t seq) {
  return (b && seq >= 0 && seq < b->max_seqs) ? b->cur_len[seq] : -1;
}

extern "C" int32_t hl_dense_batch_prefill(hl_dense_batch* b, int32_t seq, const int32_t* tokens_h, int32_t n, int32_t start_pos,
                                          float* logits_h) {
  if (!b || !d.loaded) return dfail(HL_ERR_ARG, "no model loaded or null batch");
  if (seq < 0 || seq >= b->max_seqs) return dfail(HL_ERR_ARG, "sequence index out of range");
  if (!tokens_h || !logits_h) return dfail(HL_ERR_ARG, "null argument");
  if (n <= 0) return dfail(HL_ERR_ARG, "prefill requires at least one token");
  if (start_pos < 0 || start_pos > b->cur_len[seq]) return dfail(HL_ERR_ARG, "start_pos must lie within what the sequence already holds");
  if (static_cast<int64_t>(start_pos) + n > b->max_len) return dfail(HL_ERR_CAPACITY, "prefill exceeds KV cache capacity");
  D_PASS(forward(tokens_h, n, start_pos, KvRef{b->kv, b->tables_d + static_cast<size_t>(seq) * b->nb, b->nb}, false));
  D_CUDA(cudaMemcpyAsync(logits_h, d.logits, d.hp.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, d.ctx->stream));
  D_PASS(finish());
  b->cur_len[seq] = start_pos + n;
  return HL_OK;
}

extern "C" int32_t hl_dense_batch_decode(hl_dense_batch* b, const int32_t* seq_ids_h, const int32_t* tokens_h, int32_t n_active,
                                         int32_t* next_tokens_h, float* logits_h, float* gpu_ms) {
  if (!b || !d.loaded) return dfail(HL_ERR_ARG, "no model loaded or null batch");
  if (!seq_ids_h || !tokens_h || (!next_tokens_h && !logits_h)) return dfail(HL_ERR_ARG, "null argument");
  if (n_active <= 0 || n_active > b->max_seqs) return dfail(HL_ERR_ARG, "n_active must be 1..max_seqs");
  D_CUDA(cudaSetDevice(d.device));
  const int n = n_active, nb = b->nb, S = b->max_seqs;
  cudaStream_t st = d.ctx->stream;
  D_CUDA(cudaStreamSynchronize(st));  // the pinned step record of the previous call has been consumed
  int32_t* next_h = b->pinned + 2;        // [n]
  int32_t* ctx_h = b->pinned + 2 + S;     // [n]
  int32_t* tok_h = b->pinned + 2 + 2 * S; // [n]
  int32_t* tab_h = b->pinned + 2 + 3 * S; // [n][nb]
  std::vector<char> seen(S, 0);
  int max_ctx = 0;
  for (int i = 0; i < n; ++i) {
    const int s = seq_ids_h[i];
    if (s < 0 || s >= S) return dfail(HL_ERR_ARG, "sequence index out of range");
    if (seen[s]) return dfail(HL_ERR_ARG, "a sequence appears twice in one decode step");
    seen[s] = 1;
    if (b->cur_len[s] >= b->max_len) return dfail(HL_ERR_CAPACITY, "KV cache full");
    ctx_h[i] = b->cur_len[s] + 1;
    tok_h[i] = tokens_h[i];
    max_ctx = ctx_h[i] > max_ctx ? ctx_h[i] : max_ctx;
    for (int j = 0; j < nb; ++j) tab_h[static_cast<size_t>(i) * nb + j] = s * nb + j;
  }
  // The step as a stream of work: inputs from the pinned record, every layer, argmax, results back to the record.
  // `grid_ctx` sizes the attention grid: the real maximum for a plain launch, the capacity inside a graph.
  auto enqueue = [&](int grid_ctx) -> int32_t {
    D_CUDA(cudaMemcpyAsync(b->ctx_lens_d, ctx_h, n * 4, cudaMemcpyHostToDevice, st));
    D_CUDA(cudaMemcpyAsync(b->act_tables_d, tab_h, static_cast<size_t>(n) * nb * 4, cudaMemcpyHostToDevice, st));
    BatchDecode bd{b->kv, b->ctx_lens_d, b->act_tables_d, nb, grid_ctx, b->logits_d};
    D_PASS(forward(tok_h, n, 0, KvRef{}, true, 0, false, &bd));
    argmax_partial<<<dim3(kArgmaxBlocks, n), 256, 0, st>>>(b->logits_d, d.hp.n_vocab, b->cand_v, b->cand_i);
    argmax_final<<<n, kArgmaxBlocks, 0, st>>>(b->cand_v, b->cand_i, b->next_d);
    d.ctx->launches += 2;
    D_CUDA(cudaMemcpyAsync(next_h, b->next_d, n * 4, cudaMemcpyDeviceToHost, st));
    D_CUDA(cudaMemcpyAsync(b->pinned, d.ctx->status_d, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    return HL_OK;
  };
  if (d.use_graph) {
    if (b->graphs[n] && b->graph_epoch[n] != d.buf_epoch + d.ctx->scratch_epoch) {  // a buffer it points to has moved
      cudaGraphExecDestroy(b->graphs[n]);
      b->graphs[n] = nullptr;
    }
    if (!b->graphs[n]) {
      // an uncaptured pass first (it sizes every scratch buffer; the replay repeats it with the same inputs)
      D_PASS(enqueue(b->max_len));
      D_CUDA(cudaStreamSynchronize(st));
      const int64_t counted = d.ctx->launches;
      D_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
      const int32_t rc = enqueue(b->max_len);
      cudaGraph_t graph = nullptr;
      const cudaError_t e = cudaStreamEndCapture(st, &graph);
      d.ctx->launches = counted;  // recorded, not launched
      if (rc != HL_OK || e != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        return rc != HL_OK ? rc : dfail(HL_ERR_CUDA, "stream capture of the batched decode step failed");
      }
      const cudaError_t e2 = cudaGraphInstantiate(&b->graphs[n], graph, 0);
      cudaGraphDestroy(graph);
      if (e2 != cudaSuccess) {
        b->graphs[n] = nullptr;
        return dfail(HL_ERR_CUDA, "cudaGraphInstantiate failed");
      }
      b->graph_epoch[n] = d.buf_epoch + d.ctx->scratch_epoch;  // both only ever grow, so the sum changes when either does
    }
    if (gpu_ms) D_CUDA(cudaEventRecord(d.e0, st));
    D_CUDA(cudaGraphLaunch(b->graphs[n], st));
    if (gpu_ms) D_CUDA(cudaEventRecord(d.e1, st));
  } else {
    if (gpu_ms) D_CUDA(cudaEventRecord(d.e0, st));
    D_PASS(enqueue(max_ctx));
    if (gpu_ms) D_CUDA(cudaEventRecord(d.e1, st));
  }
  if (logits_h)
    D_CUDA(cudaMemcpyAsync(logits_h, b->logits_d, static_cast<size_t>(n) * d.hp.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, st));
  D_CUDA(cudaStreamSynchronize(st));
  if (b->pinned[0] != 0) {
    const int32_t code = b->pinned[0];
    cudaMemset(d.ctx->status_d, 0, 2 * sizeof(int32_t));
    return dfail(code, "a device-side check failed during the decode step");
  }
  if (gpu_ms) D_CUDA(cudaEventElapsedTime(gpu_ms, d.e0, d.e1));
  for (int i = 0; i < n; ++i) {
    if (next_tokens_h) next_tokens_h[i] = next_h[i];
    b->cur_len[seq_ids_h[i]] += 1;
  }
  return HL_OK;
}

extern "C" int32_t hl_dense_set_decode_graph(int32_t enabled) {
  d.use_graph = enabled != 0;
  return HL_OK;
}

extern "C" const char* hl_dense_last_error(void) { return d.err.c_str(); }

extern "C" int32_t hl_dense_init_kv_cache(int32_t device, const hl_dense_hparams* hp, int32_t max_len, hl_kv_cache* out) {
  if (!out) return dfail(HL_ERR_ARG, "null cache");
  D_PASS(check_hp(hp));
  if (max_len <= 0) return dfail(HL_ERR_ARG, "max_len must be positive");
  D_PASS(ensure_ctx(device));
  const int bt = 128;  // whole 128-key tiles per page: the prefill kernel fetches them as single TMA boxes
  const int nb = (max_len + bt - 1) / bt;
  hl_kv* kv = nullptr;
  D_TRY(hl_b200_kv_create(d.ctx, hp->n_layer, hp->n_head_kv, hp->head_dim, bt, nb, &kv));
  if (d.table_len < nb) {
    // Grow-only.  A decode graph captured for an older cache has the old table address baked in: the epoch bump
    // makes the next step of that cache capture again instead of replaying through freed memory.
    if (d.table_d) cudaFree(d.table_d);
    d.table_d = nullptr;
    d.table_len = 0;
    d.buf_epoch++;
    std::vector<int32_t> ident(nb);
    for (int i = 0; i < nb; ++i) ident[i] = i;
    cudaError_t e = cudaMalloc(&d.table_d, nb * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMemcpy(d.table_d, ident.data(), nb * sizeof(int32_t), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      if (d.table_d) cudaFree(d.table_d);
      d.table_d = nullptr;
      hl_b200_kv_destroy(d.ctx, kv);
      return dfail(HL_ERR_CUDA, "block table allocation failed");
    }
    d.table_len = nb;
  }
  out->cur_len = 0;
  out->max_len = max_len;
  out->n_head_kv = hp->n_head_kv;
  out->head_dim = hp->head_dim;
  out->gpu_cache = kv;
  return HL_OK;
}

extern "C" int32_t hl_dense_free_kv_cache(hl_kv_cache* cache) {
  if (!cache || !cache->gpu_cache || !d.ctx) return dfail(HL_ERR_ARG, "null cache");
  if (d.graph && d.graph_kv == cache->gpu_cache) {
    cudaGraphExecDestroy(d.graph);
    d.graph = nullptr;
    d.graph_kv = nullptr;
  }
  hl_b200_kv_destroy(d.ctx, static_cast<hl_kv*>(cache->gpu_cache));
  cache->gpu_cache = nullptr;
  return HL_OK;
}

extern "C" int32_t hl_dense_load_model(int32_t device, const hl_dense_hparams* hp, const hl_dense_weights* w) {
  D_PASS(check_hp(hp));
  if (!w || !w->tok_emb || !w->attn_norm || !w->wq || !w->wk || !w->wv || !w->wo || !w->ffn_norm || !w->w_gate || !w->w_up ||
      !w->w_down || !w->out_norm || !w->w_out)
    return dfail(HL_ERR_ARG, "null weights");
  if (d.loaded) return dfail(HL_ERR_ARG, "a model is already loaded (one model per process)");
  D_PASS(ensure_ctx(device));
  D_CUDA(cudaSetDevice(device));
  d.hp = *hp;
  const size_t L = hp->n_layer, E = hp->n_emb, F = hp->n_ffn, V = hp->n_vocab, hd = hp->head_dim;
  const size_t qd = static_cast<size_t>(hp->n_head) * hd, kd = static_cast<size_t>(hp->n_head_kv) * hd, qkvd = qd + 2 * kd;
  // merged per-layer matrices: [Wq; Wk; Wv], and Wgate / Wup interleaved row by row, so that each group of
  // projections is one GEMM and SiLU(gate) * up can run in the epilogue of the decode projection
  std::vector<uint16_t> qkv(L * qkvd * E), gu(L * 2 * F * E);
  for (size_t l = 0; l < L; ++l) {
    memcpy(&qkv[l * qkvd * E], w->wq + l * qd * E, qd * E * 2);
    memcpy(&qkv[l * qkvd * E + qd * E], w->wk + l * kd * E, kd * E * 2);
    memcpy(&qkv[l * qkvd * E + (qd + kd) * E], w->wv + l * kd * E, kd * E * 2);
    for (size_t f = 0; f < F; ++f) {  // rows interleaved: 2f = gate_f, 2f + 1 = up_f
      memcpy(&gu[(l * 2 * F + 2 * f) * E], w->w_gate + (l * F + f) * E, E * 2);
      memcpy(&gu[(l * 2 * F + 2 * f + 1) * E], w->w_up + (l * F + f) * E, E * 2);
    }
  }
  bool ok = upload(&d.tok_emb, w->tok_emb, V * E) && upload(&d.wqkv, qkv.data(), qkv.size()) &&
            upload(&d.wo, w->wo, L * E * qd) && upload(&d.wgu, gu.data(), gu.size()) && upload(&d.wdown, w->w_down, L * E * F) &&
            upload(&d.wout, w->w_out, V * E) && upload(&d.attn_norm, w->attn_norm, L * E) &&
            upload(&d.ffn_norm, w->ffn_norm, L * E) && upload(&d.out_norm, w->out_norm, E);
  if (ok && w->q_norm) ok = upload(&d.q_norm, w->q_norm, L * hd);
  if (ok && w->k_norm) ok = upload(&d.k_norm, w->k_norm, L * hd);
  ok = ok && cudaMalloc(&d.logits, V * sizeof(float)) == cudaSuccess && cudaMalloc(&d.ctx_len_d, sizeof(int32_t)) == cudaSuccess &&
       cudaMalloc(&d.next_d, sizeof(int32_t)) == cudaSuccess && cudaMalloc(&d.cand_v, kArgmaxBlocks * sizeof(float)) == cudaSuccess &&
       cudaMalloc(&d.cand_i, kArgmaxBlocks * sizeof(int32_t)) == cudaSuccess && cudaMallocHost(&d.pinned, 8 * sizeof(int32_t)) == cudaSuccess &&
       cudaEventCreate(&d.e0) == cudaSuccess && cudaEventCreate(&d.e1) == cudaSuccess;
  d.loaded = true;  // so that unload frees whatever was allocated
  if (!ok) {
    cudaGetLastError();
    hl_dense_unload_model();
    return dfail(HL_ERR_CUDA, "weight upload failed");
  }
  const int rope_dim = hp->rope_dim > 0 ? hp->rope_dim : hp->head_dim;
  std::vector<float> theta(rope_dim / 2);
  D_TRY(hl_b200_theta_table_h(hp->rope_freq_base, rope_dim, theta.data()));
  if (hp->llama3_scaling) D_TRY(hl_b200_theta_llama3_scale_h(theta.data(), rope_dim / 2, 32.f, 1.f, 4.f, 8192));
  D_TRY(hl_b200_set_rope(d.ctx, theta.data(), rope_dim / 2));
  return HL_OK;
}

extern "C" int32_t hl_dense_unload_model(void) {
  if (!d.ctx) return HL_OK;
  cudaSetDevice(d.device);
  cudaStreamSynchronize(d.ctx->stream);
  for (__half** p : {&d.tok_emb, &d.wqkv, &d.wo, &d.wgu, &d.wdown, &d.wout, &d.xn, &d.attn, &d.gu, &d.h}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  for (float** p : {&d.attn_norm, &d.ffn_norm, &d.out_norm, &d.q_norm, &d.k_norm, &d.x, &d.qkv, &d.logits, &d.cand_v}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  for (int32_t** p : {&d.tokens_d, &d.ctx_len_d, &d.table_d, &d.next_d, &d.cand_i}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  if (d.graph) cudaGraphExecDestroy(d.graph);
  d.graph = nullptr;
  d.graph_kv = nullptr;
  if (d.pinned) cudaFreeHost(d.pinned);
  d.pinned = nullptr;
  if (d.e0) cudaEventDestroy(d.e0);
  if (d.e1) cudaEventDestroy(d.e1);
  d.e0 = d.e1 = nullptr;
  d.cap = d.table_len = 0;
  d.loaded = false;
  hl_b200_destroy(d.ctx);
  d.ctx = nullptr;
  d.device = -1;
  return HL_OK;
}

extern "C" int32_t hl_dense_forward_prefill(const int32_t* tokens_h, int32_t n, hl_kv_cache* cache, float* logits_h) {
  D_PASS(check_cache(cache));
  if (!tokens_h || !logits_h) return dfail(HL_ERR_ARG, "null argument");
  if (n <= 0) return dfail(HL_ERR_ARG, "prefill requires at least one token");
  if (n > cache->max_len) return dfail(HL_ERR_CAPACITY, "prefill exceeds KV cache capacity");
  D_PASS(forward(tokens_h, n, 0, ref_of(cache), false));
  D_CUDA(cudaMemcpyAsync(logits_h, d.logits, d.hp.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, d.ctx->stream));
  D_PASS(finish());
  cache->cur_len = n;
  return HL_OK;
}

extern "C" int32_t hl_dense_forward_prefill_chunk(const int32_t* tokens_h, int32_t n, hl_kv_cache* cache, float* logits_h) {
  D_PASS(check_cache(cache));
  if (!tokens_h || !logits_h) return dfail(HL_ERR_ARG, "null argument");
  if (n <= 0) return dfail(HL_ERR_ARG, "prefill requires at least one token");
  if (cache->cur_len < 0) return dfail(HL_ERR_ARG, "negative cur_len");
  if (static_cast<int64_t>(cache->cur_len) + n > cache->max_len) return dfail(HL_ERR_CAPACITY, "prefill exceeds KV cache capacity");
  D_PASS(forward(tokens_h, n, cache->cur_len, ref_of(cache), false));
  D_CUDA(cudaMemcpyAsync(logits_h, d.logits, d.hp.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, d.ctx->stream));
  D_PASS(finish());
  cache->cur_len += n;
  return HL_OK;
}

extern "C" int32_t hl_dense_forward_decode(int32_t token, hl_kv_cache* cache, float* logits_h) {
  D_PASS(check_cache(cache));
  if (!logits_h) return dfail(HL_ERR_ARG, "null logits");
  if (cache->cur_len >= cache->max_len) return dfail(HL_ERR_CAPACITY, "KV cache full");
  if (d.use_graph) return decode_graph(token, cache, logits_h, nullptr, nullptr);
  D_PASS(forward(&token, 1, cache->cur_len, ref_of(cache), true));
  D_CUDA(cudaMemcpyAsync(logits_h, d.logits, d.hp.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, d.ctx->stream));
  D_PASS(finish());
  cache->cur_len += 1;
  return HL_OK;
}

extern "C" int32_t hl_dense_forward_decode_token_timed(int32_t token, hl_kv_cache* cache, int32_t* next_token, float* gpu_ms) {
  D_PASS(check_cache(cache));
  if (!next_token) return dfail(HL_ERR_ARG, "null next_token");
  if (cache->cur_len >= cache->max_len) return dfail(HL_ERR_CAPACITY, "KV cache full");
  if (d.use_graph) return decode_graph(token, cache, nullptr, next_token, gpu_ms);
  if (gpu_ms) D_CUDA(cudaEventRecord(d.e0, d.ctx->stream));
  D_PASS(forward(&token, 1, cache->cur_len, ref_of(cache), true));
  launch_argmax(d.ctx->stream);
  if (gpu_ms) D_CUDA(cudaEventRecord(d.e1, d.ctx->stream));
  D_CUDA(cudaMemcpyAsync(&d.pinned[2], d.next_d, sizeof(int32_t), cudaMemcpyDeviceToHost, d.ctx->stream));
  D_PASS(finish());
  if (gpu_ms) D_CUDA(cudaEventElapsedTime(gpu_ms, d.e0, d.e1));
  *next_token = d.pinned[2];
  cache->cur_len += 1;
  return HL_OK;
}
