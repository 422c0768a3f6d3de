// The reference's backend contract over the B200 attention path (C ABI in include/hl_backend.h),
// with an attention-only stand-in model around it.  The orchestration mirrors the order of
// operations of forwardPrefill / forwardDecode (src/hippo_leap/backends/naive.nim:4063-4078,
// 4697-4717): per layer  Q/K/V rows -> [QK-norm -> RoPE -> KV store -> attention]  -> logits.
// The bracketed part is the product path (libhl_b200 entry points); the row lookup and the logits
// product around it are plain glue kernels.
#include <cuda_runtime.h>
#include <math.h>

#include <string>
#include <vector>

#include "../../include/hl_backend.h"
#include "host_common.h"

namespace {

struct Backend {
  hl_ctx* ctx = nullptr;
  int device = -1;
  bool loaded = false;
  hl_hparams hp{};
  float *eq = nullptr, *ek = nullptr, *ev = nullptr, *wout = nullptr, *qn = nullptr, *kn = nullptr;
  float *q = nullptr, *k = nullptr, *v = nullptr, *out = nullptr;  // activations [cap][dim]
  int act_cap = 0;
  float* logits_d = nullptr;
  int32_t* tokens_d = nullptr;
  int tokens_cap = 0;
  int32_t* ctx_len_d = nullptr;  // one-sequence ctx_lens for the decode step
  int32_t* table_d = nullptr;    // identity block table of the single sequence
  int table_len = 0;
  int32_t* next_d = nullptr;
  int32_t* status_h = nullptr;  // pinned copy of the device status word
  int32_t* step_h = nullptr;    // pinned {token id, ctx_len, next token}: inputs / output of the replayed decode graph
  cudaGraphExec_t graph = nullptr;  // one decode step (all layers) captured once per (cache, max_len)
  const void* graph_kv = nullptr;
  int graph_max_len = 0;
  uint64_t buf_epoch = 0;                             // bumped when an activation / token buffer is re-allocated
  uint64_t graph_buf_epoch = 0, graph_ctx_epoch = 0;  // what the captured graph was recorded against
  bool use_graph = true;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  std::string err;
} g;

int32_t bfail(int32_t code, const char* msg) {
  g.err = msg;
  return code;
}
int32_t bfail_ctx(int32_t code, const char* call) {
  const char* inner = g.ctx ? hl_b200_last_error(g.ctx) : "";
  g.err = (inner && *inner) ? std::string(inner) : std::string(call) + " failed";
  return code;
}
#define B_CUDA(expr)                                                    \
  do {                                                                  \
    cudaError_t e_ = (expr);                                            \
    if (e_ != cudaSuccess) return bfail(HL_ERR_CUDA, cudaGetErrorString(e_)); \
  } while (0)
// B_TRY wraps a libhl_b200 call (its message comes from the context); B_PASS forwards the status of a
// backend helper that has already recorded its own message.
#define B_TRY(expr)                          \
  do {                                       \
    int32_t rc_ = (expr);                    \
    if (rc_ != HL_OK) return bfail_ctx(rc_, #expr); \
  } while (0)
#define B_PASS(expr)              \
  do {                            \
    int32_t rc_ = (expr);         \
    if (rc_ != HL_OK) return rc_; \
  } while (0)

int32_t ensure_ctx(int device) {
  if (g.ctx) return device == g.device ? HL_OK : bfail(HL_ERR_ARG, "backend already bound to another device");
  int32_t rc = hl_b200_create(device, nullptr, &g.ctx);
  if (rc != HL_OK) return bfail(rc, "hl_b200_create failed: no usable sm_100 device (no CPU fallback exists)");
  g.device = device;
  // this backend always queues the KV append between the kernel that produces the query rows and the attention kernel:
  // the attention kernels may start their query prologue while the append runs
  g.ctx->chain_pdl = true;
  return HL_OK;
}

// the three lookups of one layer in one launch: blockIdx.y = 0 / 1 / 2 selects q / k / v
__global__ void gather_qkv_kernel(const float* __restrict__ eq, const float* __restrict__ ek,
                                  const float* __restrict__ ev, const int32_t* __restrict__ tokens, int qd, int kd,
                                  int n_vocab, float* __restrict__ q, float* __restrict__ k, float* __restrict__ v) {
  const int t = blockIdx.x, which = blockIdx.y;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= n_vocab ? n_vocab - 1 : tok);
  const int dim = which == 0 ? qd : kd;
  const float* table = which == 0 ? eq : (which == 1 ? ek : ev);
  float* dst = which == 0 ? q : (which == 1 ? k : v);
  const float4* src = reinterpret_cast<const float4*>(table + static_cast<int64_t>(tok) * dim);
  float4* d = reinterpret_cast<float4*>(dst + static_cast<int64_t>(t) * dim);
  for (int i = threadIdx.x; i < dim / 4; i += blockDim.x) d[i] = src[i];
}

// x = sum over layers of the last token's attention output (layer order, float32 adds);
// logits[v] = sum_d x[d] * wout[d][v], d ascending, separate multiply and add (no FMA contraction),
// i.e. the k-innermost float32 accumulation of the reference's CPU matmul (tensor.nim:77-80).
//
// One thread owns one logit and adds its q_dim products strictly in order (that order is the result), so a block
// cannot split the sum; what it can do is feed it: a block of 256 threads serves 32 logits, all 256 fetch the next
// [64 d][32 v] tile of wout (coalesced 128-byte rows, eight loads in flight per thread) while the 32 owning threads
// run down the current tile in shared memory.  (With one logit per thread and nothing else -- two blocks for a
// 512-word vocabulary -- each warp had four loads in flight and the projection took longer than all sixteen attention
// layers of a decode step together.)
constexpr int kLogitsV = 32, kLogitsD = 64;
__global__ void __launch_bounds__(256) logits_kernel(const float* __restrict__ outs, int n_layer, int64_t layer_stride,
                                                     int q_dim, const float* __restrict__ wout, int n_vocab,
                                                     float* __restrict__ logits) {
  extern __shared__ float x[];                       // [q_dim] summed layer outputs
  __shared__ float tile[2][kLogitsD][kLogitsV];      // two tiles of wout, 8 KiB each
  for (int d = threadIdx.x; d < q_dim; d += blockDim.x) {
    float acc = outs[d];
    for (int l = 1; l < n_layer; ++l) acc = __fadd_rn(acc, outs[l * layer_stride + d]);
    x[d] = acc;
  }
  const int v0 = blockIdx.x * kLogitsV;
  const int c = threadIdx.x % kLogitsV, r0 = threadIdx.x / kLogitsV;  // this thread loads column c of rows r0, r0 + 8, ...
  const bool col_ok = v0 + c < n_vocab;
  float reg[kLogitsD / 8];
  auto fetch = [&](int d0) {
#pragma unroll
    for (int i = 0; i < kLogitsD / 8; ++i) {
      const int d = d0 + r0 + 8 * i;
      reg[i] = (col_ok && d < q_dim) ? wout[static_cast<int64_t>(d) * n_vocab + v0 + c] : 0.f;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < kLogitsD / 8; ++i) tile[buf][r0 + 8 * i][c] = reg[i];
  };
  fetch(0);
  stash(0);
  __syncthreads();  // x and the first tile are in place
  float acc = 0.f;
  int buf = 0;
  for (int d0 = 0; d0 < q_dim; d0 += kLogitsD) {
    const bool more = d0 + kLogitsD < q_dim;
    if (more) fetch(d0 + kLogitsD);                  // in flight while the owners add
    if (threadIdx.x < kLogitsV) {
      const int n = min(kLogitsD, q_dim - d0);
      if (n == kLogitsD) {  // whole tile: unrolled, so the shared-memory loads run ahead of the chain of additions
#pragma unroll
        for (int d = 0; d < kLogitsD; ++d) acc = __fadd_rn(acc, __fmul_rn(x[d0 + d], tile[buf][d][threadIdx.x]));
      } else {
        for (int d = 0; d < n; ++d) acc = __fadd_rn(acc, __fmul_rn(x[d0 + d], tile[buf][d][threadIdx.x]));
      }
    }
    if (more) stash(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }
  if (threadIdx.x < kLogitsV && v0 + threadIdx.x < n_vocab) logits[v0 + threadIdx.x] = acc;
}

// first maximal index wins, as argmaxLast (src/hippo_leap/sampling.nim:13-19)
__global__ void argmax_first_kernel(const float* __restrict__ logits, int n, int32_t* __restrict__ out) {
  __shared__ float bv[256];
  __shared__ int bi[256];
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = logits[i];
    if (v > best || (v == best && i < idx)) {
      best = v;
      idx = i;
    }
  }
  bv[threadIdx.x] = best;
  bi[threadIdx.x] = idx;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float ov = bv[threadIdx.x + s];
      const int oi = bi[threadIdx.x + s];
      if (ov > bv[threadIdx.x] || (ov == bv[threadIdx.x] && oi < bi[threadIdx.x])) {
        bv[threadIdx.x] = ov;
        bi[threadIdx.x] = oi;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *out = bi[0];
}

__global__ void set_i32_kernel(int32_t* p, int32_t v) { *p = v; }

int32_t check_hp(const hl_hparams* hp) {
  if (!hp) return bfail(HL_ERR_ARG, "null hparams");
  if (hp->n_head <= 0 && hp->n_layer > 0) return bfail(HL_ERR_ARG, "model requires head_count or SSM parameters");
  if (hp->n_vocab <= 0 || hp->n_layer <= 0 || hp->n_head_kv <= 0) return bfail(HL_ERR_ARG, "non-positive hparam");
  if (hp->n_head % hp->n_head_kv != 0) return bfail(HL_ERR_ARG, "GQA requires head_count divisible by head_count_kv");
  if (hp->head_dim != 64 && hp->head_dim != 128 && hp->head_dim != 256)
    return bfail(HL_ERR_UNSUPPORTED, "head_dim must be 64, 128 or 256");
  return HL_OK;
}

int32_t ensure_act(int n_tok) {
  if (n_tok <= g.act_cap) return HL_OK;
  cudaStreamSynchronize(g.ctx->stream);
  for (float** p : {&g.q, &g.k, &g.v, &g.out}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  g.act_cap = 0;
  g.buf_epoch++;
  const size_t qd = static_cast<size_t>(g.hp.n_head) * g.hp.head_dim, kd = static_cast<size_t>(g.hp.n_head_kv) * g.hp.head_dim;
  B_CUDA(cudaMalloc(&g.q, n_tok * qd * sizeof(float)));
  B_CUDA(cudaMalloc(&g.k, n_tok * kd * sizeof(float)));
  B_CUDA(cudaMalloc(&g.v, n_tok * kd * sizeof(float)));
  B_CUDA(cudaMalloc(&g.out, static_cast<size_t>(g.hp.n_layer) * n_tok * qd * sizeof(float)));
  g.act_cap = n_tok;
  return HL_OK;
}

hl_attn_shape shape_for_layer(int l) {
  hl_attn_shape s{};
  s.n_head = g.hp.n_head;
  s.n_head_kv = g.hp.n_head_kv;
  s.head_dim = g.hp.head_dim;
  s.rope_dim = g.hp.rope_dim > 0 ? g.hp.rope_dim : g.hp.head_dim;  // naive.nim:3979
  s.rope_mode = g.hp.rope_mode;
  s.rms_eps = g.hp.rms_eps;
  s.q_norm_w = g.qn ? g.qn + static_cast<size_t>(l) * g.hp.head_dim : nullptr;
  s.k_norm_w = g.kn ? g.kn + static_cast<size_t>(l) * g.hp.head_dim : nullptr;
  return s;
}

// One forward over n tokens starting at position pos0; decode is n == 1.
// `grid_ctx` sizes the decode grid and scratch (>= the real context); with `from_step_h` the token id and
// the context length are read from the pinned step buffer by copy nodes, so that a captured graph of
// this sequence can be replayed for every token (the reference's megakernel backend replays a HIP
// graph fed by a device-side step record the same way: backends/megakernel.nim:78-83, 2458-2479).
int32_t forward(const int32_t* tokens_h, int n, int pos0, hl_kv_cache* cache, bool decode, int grid_ctx = 0,
                bool from_step_h = false) {
  hl_kv* kv = static_cast<hl_kv*>(cache->gpu_cache);
  const int qd = g.hp.n_head * g.hp.head_dim, kd = g.hp.n_head_kv * g.hp.head_dim;
  B_CUDA(cudaSetDevice(g.device));
  if (ensure_act(n) != HL_OK) return HL_ERR_CUDA;
  if (n > g.tokens_cap) {
    cudaStreamSynchronize(g.ctx->stream);
    if (g.tokens_d) cudaFree(g.tokens_d);
    g.tokens_d = nullptr;
    g.buf_epoch++;
    B_CUDA(cudaMalloc(&g.tokens_d, n * sizeof(int32_t)));
    g.tokens_cap = n;
  }
  cudaStream_t st = g.ctx->stream;
  if (from_step_h) {
    B_CUDA(cudaMemcpyAsync(g.tokens_d, &g.step_h[0], sizeof(int32_t), cudaMemcpyHostToDevice, st));
    B_CUDA(cudaMemcpyAsync(g.ctx_len_d, &g.step_h[1], sizeof(int32_t), cudaMemcpyHostToDevice, st));
  } else {
    B_CUDA(cudaMemcpyAsync(g.tokens_d, tokens_h, n * sizeof(int32_t), cudaMemcpyHostToDevice, st));
    if (decode) {
      set_i32_kernel<<<1, 1, 0, st>>>(g.ctx_len_d, pos0 + 1);
      g.ctx->launches += 1;
    }
  }
  if (grid_ctx < pos0 + 1) grid_ctx = pos0 + 1;
  const int64_t layer_stride = static_cast<int64_t>(g.act_cap) * qd;
  for (int l = 0; l < g.hp.n_layer; ++l) {
    const size_t toff = static_cast<size_t>(l) * g.hp.n_vocab;
    gather_qkv_kernel<<<dim3(n, 3), 128, 0, st>>>(g.eq + toff * qd, g.ek + toff * kd, g.ev + toff * kd, g.tokens_d, qd,
                                                   kd, g.hp.n_vocab, g.q, g.k, g.v);
    g.ctx->launches += 1;
    const hl_attn_shape s = shape_for_layer(l);
    hl_view qv{g.q, HL_DTYPE_F32, qd, g.hp.head_dim, 1}, kv_{g.k, HL_DTYPE_F32, kd, g.hp.head_dim, 1},
        vv{g.v, HL_DTYPE_F32, kd, g.hp.head_dim, 1}, ov{g.out + l * layer_stride, HL_DTYPE_F32, qd, g.hp.head_dim, 1};
    if (decode) {
      B_TRY(hl_b200_kv_append_batch(g.ctx, kv, l, &s, &kv_, &vv, 1, g.ctx_len_d, g.table_d, kv->num_blocks));
      B_TRY(hl_b200_attn_decode(g.ctx, kv, l, &s, &qv, 1, g.ctx_len_d, grid_ctx, g.table_d, kv->num_blocks, &ov, nullptr));
    } else {
      B_TRY(hl_b200_kv_append_seq(g.ctx, kv, l, &s, &kv_, &vv, n, pos0, g.table_d, kv->num_blocks));
      B_TRY(hl_b200_attn_prefill(g.ctx, kv, l, &s, &qv, n, pos0, g.table_d, kv->num_blocks, &ov, nullptr));
    }
  }
  logits_kernel<<<(g.hp.n_vocab + kLogitsV - 1) / kLogitsV, 256, qd * sizeof(float), st>>>(
      g.out + static_cast<int64_t>(n - 1) * qd, g.hp.n_layer, layer_stride, qd, g.wout, g.hp.n_vocab, g.logits_d);
  g.ctx->launches += 1;
  B_CUDA(cudaGetLastError());
  return HL_OK;
}

// One synchronisation per forward call, like the reference (naive.nim:4584, 5081): the result
// copy queued by the caller and the device status word arrive together.
int32_t finish_status() {
  B_CUDA(cudaMemcpyAsync(g.status_h, g.ctx->status_d, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, g.ctx->stream));
  B_CUDA(cudaStreamSynchronize(g.ctx->stream));
  if (g.status_h[0] != 0) {
    const int32_t code = g.status_h[0];
    cudaMemset(g.ctx->status_d, 0, 2 * sizeof(int32_t));
    return bfail(code, code == HL_ERR_TIMEOUT ? "a bounded device-side wait gave up during the forward pass"
                                              : "a device-side index check failed during the forward pass");
  }
  return HL_OK;
}

int32_t check_cache(const hl_kv_cache* cache) {
  if (!g.loaded) return bfail(HL_ERR_ARG, "no model loaded (loadModelBackend)");
  if (!cache || !cache->gpu_cache) return bfail(HL_ERR_ARG, "null KV cache (initKvCache)");
  return HL_OK;
}

}  // namespace

extern "C" const char* hl_backend_last_error(void) { return g.err.c_str(); }
extern "C" int64_t hl_backend_launch_count(void) { return g.ctx ? g.ctx->launches : 0; }

extern "C" int32_t hl_backend_init_kv_cache(int32_t device, const hl_hparams* hp, int32_t max_len, hl_kv_cache* out) {
  if (!out) return bfail(HL_ERR_ARG, "null cache");
  B_PASS(check_hp(hp));
  if (max_len <= 0) return bfail(HL_ERR_ARG, "max_len must be positive");
  B_PASS(ensure_ctx(device));
  const int bt = 16;
  const int nb = (max_len + bt - 1) / bt;
  hl_kv* kv = nullptr;
  B_TRY(hl_b200_kv_create(g.ctx, hp->n_layer, hp->n_head_kv, hp->head_dim, bt, nb, &kv));
  if (g.table_len < nb) {
    // Grow-only identity table shared by all caches (each uses its own number of blocks as the length).  A decode
    // graph captured for an older cache has the old address baked in: the epoch bump makes it capture again.
    if (g.table_d) cudaFree(g.table_d);
    g.table_d = nullptr;
    g.table_len = 0;
    g.buf_epoch++;
    std::vector<int32_t> ident(nb);
    for (int i = 0; i < nb; ++i) ident[i] = i;
    cudaError_t e = cudaMalloc(&g.table_d, nb * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMemcpy(g.table_d, ident.data(), nb * sizeof(int32_t), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      if (g.table_d) cudaFree(g.table_d);
      g.table_d = nullptr;
      hl_b200_kv_destroy(g.ctx, kv);
      return bfail(HL_ERR_CUDA, "block table allocation failed");
    }
    g.table_len = nb;
  }
  out->cur_len = 0;
  out->max_len = max_len;
  out->n_head_kv = hp->n_head_kv;
  out->head_dim = hp->head_dim;
  out->gpu_cache = kv;
  return HL_OK;
}

extern "C" int32_t hl_backend_free_kv_cache(hl_kv_cache* cache) {
  if (!cache || !cache->gpu_cache || !g.ctx) return bfail(HL_ERR_ARG, "null cache");
  hl_b200_kv_destroy(g.ctx, static_cast<hl_kv*>(cache->gpu_cache));
  cache->gpu_cache = nullptr;
  return HL_OK;
}

extern "C" int32_t hl_backend_load_model(int32_t device, const hl_hparams* hp, const hl_standin_weights* w) {
  B_PASS(check_hp(hp));
  if (!w || !w->eq || !w->ek || !w->ev || !w->wout) return bfail(HL_ERR_ARG, "null weights");
  if (g.loaded) return bfail(HL_ERR_ARG, "a model is already loaded (one model per process)");
  B_PASS(ensure_ctx(device));
  B_CUDA(cudaSetDevice(device));
  g.hp = *hp;
  const size_t qd = static_cast<size_t>(hp->n_head) * hp->head_dim, kd = static_cast<size_t>(hp->n_head_kv) * hp->head_dim;
  const size_t lv = static_cast<size_t>(hp->n_layer) * hp->n_vocab;
  auto up = [&](float** dst, const float* src, size_t n) -> bool {
    return cudaMalloc(dst, n * sizeof(float)) == cudaSuccess &&
           cudaMemcpy(*dst, src, n * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess;
  };
  bool ok = up(&g.eq, w->eq, lv * qd) && up(&g.ek, w->ek, lv * kd) && up(&g.ev, w->ev, lv * kd) &&
            up(&g.wout, w->wout, qd * hp->n_vocab);
  if (ok && w->q_norm) ok = up(&g.qn, w->q_norm, static_cast<size_t>(hp->n_layer) * hp->head_dim);
  if (ok && w->k_norm) ok = up(&g.kn, w->k_norm, static_cast<size_t>(hp->n_layer) * hp->head_dim);
  ok = ok && cudaMalloc(&g.logits_d, hp->n_vocab * sizeof(float)) == cudaSuccess &&
       cudaMalloc(&g.ctx_len_d, sizeof(int32_t)) == cudaSuccess && cudaMalloc(&g.next_d, sizeof(int32_t)) == cudaSuccess &&
       cudaMallocHost(&g.status_h, 2 * sizeof(int32_t)) == cudaSuccess &&
       cudaMallocHost(&g.step_h, 4 * sizeof(int32_t)) == cudaSuccess && cudaEventCreate(&g.e0) == cudaSuccess &&
       cudaEventCreate(&g.e1) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    g.loaded = true;  // so that unload frees the partial state
    hl_backend_unload_model();
    return bfail(HL_ERR_CUDA, "weight upload failed");
  }
  // theta table on the host, as ensureModelGpuPtrs does (naive.nim:3850-3861)
  const int rope_dim = hp->rope_dim > 0 ? hp->rope_dim : hp->head_dim;
  std::vector<float> theta(rope_dim / 2);
  B_TRY(hl_b200_theta_table_h(hp->rope_freq_base, rope_dim, theta.data()));
  if (hp->llama3_scaling) B_TRY(hl_b200_theta_llama3_scale_h(theta.data(), rope_dim / 2, 32.f, 1.f, 4.f, 8192));
  B_TRY(hl_b200_set_rope(g.ctx, theta.data(), rope_dim / 2));
  g.loaded = true;
  return HL_OK;
}

extern "C" int32_t hl_backend_unload_model(void) {
  if (!g.ctx) return HL_OK;
  cudaSetDevice(g.device);
  cudaStreamSynchronize(g.ctx->stream);
  for (float** p : {&g.eq, &g.ek, &g.ev, &g.wout, &g.qn, &g.kn, &g.q, &g.k, &g.v, &g.out, &g.logits_d}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  for (int32_t** p : {&g.tokens_d, &g.ctx_len_d, &g.table_d, &g.next_d}) {
    if (*p) cudaFree(*p);
    *p = nullptr;
  }
  if (g.status_h) cudaFreeHost(g.status_h);
  g.status_h = nullptr;
  if (g.step_h) cudaFreeHost(g.step_h);
  g.step_h = nullptr;
  if (g.graph) cudaGraphExecDestroy(g.graph);
  g.graph = nullptr;
  g.graph_kv = nullptr;
  if (g.e0) cudaEventDestroy(g.e0);
  if (g.e1) cudaEventDestroy(g.e1);
  g.e0 = g.e1 = nullptr;
  g.act_cap = g.tokens_cap = g.table_len = 0;
  g.loaded = false;
  hl_b200_destroy(g.ctx);
  g.ctx = nullptr;
  g.device = -1;
  return HL_OK;
}

extern "C" int32_t hl_backend_forward_prefill(const int32_t* tokens_h, int32_t n, hl_kv_cache* cache, float* logits_h) {
  B_PASS(check_cache(cache));
  if (!tokens_h || !logits_h) return bfail(HL_ERR_ARG, "null argument");
  if (n <= 0) return bfail(HL_ERR_ARG, "prefill requires at least one token");
  if (n > cache->max_len) return bfail(HL_ERR_CAPACITY, "prefill exceeds KV cache capacity");
  B_PASS(forward(tokens_h, n, 0, cache, false));
  B_CUDA(cudaMemcpyAsync(logits_h, g.logits_d, g.hp.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, g.ctx->stream));
  B_PASS(finish_status());
  cache->cur_len = n;
  return HL_OK;
}

extern "C" int32_t hl_backend_forward_prefill_chunk(const int32_t* tokens_h, int32_t n, hl_kv_cache* cache, float* logits_h) {
  B_PASS(check_cache(cache));
  if (!tokens_h || !logits_h) return bfail(HL_ERR_ARG, "null argument");
  if (n <= 0) return bfail(HL_ERR_ARG, "prefill requires at least one token");
  if (cache->cur_len < 0) return bfail(HL_ERR_ARG, "negative cur_len");
  if (static_cast<int64_t>(cache->cur_len) + n > cache->max_len) return bfail(HL_ERR_CAPACITY, "prefill exceeds KV cache capacity");
  B_PASS(forward(tokens_h, n, cache->cur_len, cache, false));
  B_CUDA(cudaMemcpyAsync(logits_h, g.logits_d, g.hp.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, g.ctx->stream));
  B_PASS(finish_status());
  cache->cur_len += n;
  return HL_OK;
}

static int32_t decode_common(int32_t token, hl_kv_cache* cache) {
  B_PASS(check_cache(cache));
  if (cache->cur_len >= cache->max_len) return bfail(HL_ERR_CAPACITY, "KV cache full");
  if (cache->cur_len < 0) return bfail(HL_ERR_ARG, "negative cur_len");
  return forward(&token, 1, cache->cur_len, cache, true);
}

extern "C" int32_t hl_backend_forward_decode(int32_t token, hl_kv_cache* cache, float* logits_h) {
  if (!logits_h) return bfail(HL_ERR_ARG, "null logits");
  B_PASS(decode_common(token, cache));
  B_CUDA(cudaMemcpyAsync(logits_h, g.logits_d, g.hp.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, g.ctx->stream));
  B_PASS(finish_status());
  cache->cur_len += 1;
  return HL_OK;
}

// Capture one whole decode step (every layer + logits + argmax + the result copies) into a CUDA graph.
// The grid and the split-KV scratch are sized for the cache's full capacity, so the same graph serves
// every position: CTAs of chunks beyond the current context exit at once.
static int32_t ensure_decode_graph(hl_kv_cache* cache) {
  // still valid: same cache, and no buffer whose address the graph holds has been re-allocated since
  if (g.graph && g.graph_kv == cache->gpu_cache && g.graph_max_len == cache->max_len && g.graph_buf_epoch == g.buf_epoch &&
      g.graph_ctx_epoch == g.ctx->scratch_epoch)
    return HL_OK;
  if (g.graph) cudaGraphExecDestroy(g.graph);
  g.graph = nullptr;
  cudaStream_t st = g.ctx->stream;
  // An uncaptured pass first: it configures the kernels and grows every scratch buffer to its final size,
  // so nothing allocates or synchronises while the stream is being captured.  It runs at the caller's
  // current position and is simply repeated by the first replay (same position, same values).
  B_PASS(forward(nullptr, 1, g.step_h[1] - 1, cache, true, cache->max_len, true));
  B_CUDA(cudaStreamSynchronize(st));
  B_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
  int32_t rc = forward(nullptr, 1, g.step_h[1] - 1, cache, true, cache->max_len, true);
  if (rc == HL_OK) {
    argmax_first_kernel<<<1, 256, 0, st>>>(g.logits_d, g.hp.n_vocab, g.next_d);
    g.ctx->launches += 1;
    cudaMemcpyAsync(&g.step_h[2], g.next_d, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
    cudaMemcpyAsync(g.status_h, g.ctx->status_d, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  }
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(st, &graph);
  if (rc != HL_OK) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (e != cudaSuccess || !graph) return bfail(HL_ERR_CUDA, "stream capture of the decode step failed");
  e = cudaGraphInstantiate(&g.graph, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return bfail(HL_ERR_CUDA, "cudaGraphInstantiate failed");
  g.graph_kv = cache->gpu_cache;
  g.graph_max_len = cache->max_len;
  g.graph_buf_epoch = g.buf_epoch;
  g.graph_ctx_epoch = g.ctx->scratch_epoch;
  return HL_OK;
}

static int32_t decode_token_graph(int32_t token, hl_kv_cache* cache, int32_t* next_token, float* gpu_ms) {
  B_PASS(check_cache(cache));
  if (cache->cur_len >= cache->max_len) return bfail(HL_ERR_CAPACITY, "KV cache full");
  if (cache->cur_len < 0) return bfail(HL_ERR_ARG, "negative cur_len");
  B_CUDA(cudaSetDevice(g.device));
  g.step_h[0] = token;
  g.step_h[1] = cache->cur_len + 1;
  B_PASS(ensure_decode_graph(cache));
  cudaStream_t st = g.ctx->stream;
  if (gpu_ms) B_CUDA(cudaEventRecord(g.e0, st));
  B_CUDA(cudaGraphLaunch(g.graph, st));
  if (gpu_ms) B_CUDA(cudaEventRecord(g.e1, st));
  B_CUDA(cudaStreamSynchronize(st));
  g.ctx->launches += 3 * g.hp.n_layer + g.hp.n_layer + 2;  // kernels inside one replay (combine counted once per layer)
  if (g.status_h[0] != 0) {
    const int32_t code = g.status_h[0];
    cudaMemset(g.ctx->status_d, 0, 2 * sizeof(int32_t));
    return bfail(code, "a device-side check failed during the decode step");
  }
  if (gpu_ms) B_CUDA(cudaEventElapsedTime(gpu_ms, g.e0, g.e1));
  *next_token = g.step_h[2];
  cache->cur_len += 1;
  return HL_OK;
}

extern "C" int32_t hl_backend_set_decode_graph(int32_t enabled) {
  g.use_graph = enabled != 0;
  return HL_OK;
}

extern "C" int32_t hl_backend_forward_decode_token_timed(int32_t token, hl_kv_cache* cache, int32_t* next_token,
                                                         float* gpu_ms) {
  if (!next_token) return bfail(HL_ERR_ARG, "null next_token");
  if (g.use_graph && g.loaded) return decode_token_graph(token, cache, next_token, gpu_ms);
  B_PASS(check_cache(cache));
  if (gpu_ms) B_CUDA(cudaEventRecord(g.e0, g.ctx->stream));
  B_PASS(decode_common(token, cache));
  argmax_first_kernel<<<1, 256, 0, g.ctx->stream>>>(g.logits_d, g.hp.n_vocab, g.next_d);
  g.ctx->launches += 1;
  if (gpu_ms) B_CUDA(cudaEventRecord(g.e1, g.ctx->stream));
  B_CUDA(cudaMemcpyAsync(next_token, g.next_d, sizeof(int32_t), cudaMemcpyDeviceToHost, g.ctx->stream));
  B_PASS(finish_status());
  if (gpu_ms) B_CUDA(cudaEventElapsedTime(gpu_ms, g.e0, g.e1));
  cache->cur_len += 1;
  return HL_OK;
}

extern "C" int32_t hl_backend_forward_decode_token(int32_t token, hl_kv_cache* cache, int32_t* next_token) {
  return hl_backend_forward_decode_token_timed(token, cache, next_token, nullptr);
}
