// hl_b200_attn_decode_static: the split-KV decode step for callers that must not allocate.
//
// Who needs this: a serving loop that has handed every byte of device memory to its own KV pool or
// arena (so a cudaMalloc in steady state can simply fail), and latency-critical decode loops that
// cannot afford cudaMalloc / cudaFree at all, because both synchronise the whole device and stall every
// other stream.  hl_b200_attn_decode grows its split-KV scratch with cudaMalloc the first time a
// larger batch or context arrives; this variant never does.  Its scratch is the fixed array below,
// which lives in the library image: every GPU that loads libhl_b200.so holds it (16.25 MiB) until the
// process exits, whether or not this entry point is ever called.
//
// The price is a hard limit: batch * n_head * chunks <= kStaticTriples, where chunks is the number of
// context chunks the grid uses (ceil(max_ctx_h / chunk_tokens)); larger requests are rejected with
// HL_ERR_CAPACITY before anything is launched.
//
// Sharing: every call, on every context and stream of the process, uses the same array on a given
// GPU.  Two calls whose kernels overlap on the GPU race on it and corrupt each other's partial
// results; serialise them (one stream, or an event between streams).  The array keeps what the last
// call wrote.  That is harmless here: the decode kernel writes every (sequence, head, chunk) slot of
// the current call before the combine pass reads it, and no slot is accumulated into, so nothing has
// to start at zero and nothing is cleared.
//
// Set-up: the first call on each device looks the array's device address up with
// cudaGetSymbolAddress (in host code the array's name is only a stand-in, not a device pointer) and
// raises the kernel's shared-memory limit.  Make that first call during start-up, before any stream
// capture begins.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>

#include "../../include/hl_b200.h"
#include "attn_decode.cuh"
#include "host_common.h"

namespace {

constexpr size_t kStaticTriples = 32768;  // (sequence, head, chunk) partial slots
static __device__ __align__(256) float g_static_part_o[kStaticTriples * 128];  // 16 MiB
static __device__ __align__(256) float g_static_part_ml[kStaticTriples * 2];   // 256 KiB

constexpr int kMaxDevices = 64;
float* g_part_o_addr[kMaxDevices] = {};
float* g_part_ml_addr[kMaxDevices] = {};
bool g_smem_configured[kMaxDevices][2] = {};

// Once per device, with that device current: resolve the device addresses of the arrays.
int32_t static_setup(hl_ctx* ctx) {
  const int dev = ctx->device;
  if (dev < 0 || dev >= kMaxDevices) return hl_fail(ctx, HL_ERR_UNSUPPORTED, "device index %d beyond %d", dev, kMaxDevices);
  if (g_part_o_addr[dev] != nullptr) return HL_OK;
  void* po = nullptr;
  void* pm = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&po, g_static_part_o);
  if (e != cudaSuccess)
    return hl_fail(ctx, HL_ERR_CUDA, "cudaGetSymbolAddress(g_static_part_o) failed: %s", cudaGetErrorString(e));
  e = cudaGetSymbolAddress(&pm, g_static_part_ml);
  if (e != cudaSuccess)
    return hl_fail(ctx, HL_ERR_CUDA, "cudaGetSymbolAddress(g_static_part_ml) failed: %s", cudaGetErrorString(e));
  g_part_ml_addr[dev] = static_cast<float*>(pm);
  g_part_o_addr[dev] = static_cast<float*>(po);
  return HL_OK;
}

template <int HD>
int32_t launch(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl::DecodeArgs& a, int32_t batch) {
  using namespace hl;
  constexpr int NW = 4, STAGES = HD == 128 ? 3 : 4;
  using Cfg = DecodeCfg<HD, NW, STAGES>;
  auto kern = attn_decode_kernel<HD, NW, STAGES>;
  bool& configured = g_smem_configured[ctx->device][HD == 128 ? 1 : 0];
  if (!configured) {
    HL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  dim3 grid(a.max_chunks, a.n_head_kv, batch);
  kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, ctx->stream>>>(kv->k_map[layer], kv->v_map[layer], a);
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  if (a.max_chunks > 1) {
    attn_combine_kernel<HD><<<dim3(a.n_head, batch), HD, 0, ctx->stream>>>(a);
    ctx->launches++;
    HL_CUDA(ctx, cudaGetLastError());
  }
  return HL_OK;
}

}  // namespace

extern "C" int32_t hl_b200_attn_decode_static(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s,
                                              const hl_view* q, int32_t batch, const int32_t* ctx_lens,
                                              int32_t max_ctx_h, const int32_t* block_tables,
                                              int32_t max_blocks_per_seq, const hl_view* out) {
  // The same argument checks as hl_b200_attn_decode, so a bad view comes back as a status code, never as a fault.
  int32_t rc = hl_check_shape(ctx, kv, s, layer);
  if (rc == HL_OK) rc = hl_check_view(ctx, q, "q");
  if (rc == HL_OK) rc = hl_check_view(ctx, out, "out");
  if (rc != HL_OK) return rc;
  if (batch <= 0 || batch > 65535) return hl_fail(ctx, HL_ERR_ARG, "decode_static: batch %d outside [1, 65535]", batch);
  if (!ctx_lens || !block_tables || max_blocks_per_seq <= 0)
    return hl_fail(ctx, HL_ERR_ARG, "decode_static: null ctx_lens or block table");
  if (max_ctx_h <= 0) return hl_fail(ctx, HL_ERR_ARG, "decode_static: max_ctx_h must be positive");
  if (static_cast<int64_t>(max_ctx_h) > static_cast<int64_t>(max_blocks_per_seq) * kv->block_tokens)
    return hl_fail(ctx, HL_ERR_CAPACITY, "KV cache full: context %d exceeds the block table", max_ctx_h);
  if (s->n_head / s->n_head_kv > 16) return hl_fail(ctx, HL_ERR_UNSUPPORTED, "decode_static: n_head / n_head_kv > 16");
  HL_CUDA(ctx, cudaSetDevice(ctx->device));
  rc = static_setup(ctx);
  if (rc != HL_OK) return rc;

  hl::DecodeArgs a{};
  // the chunking rule of hl_b200_attn_decode itself: both entry points cut a context the same way, so their results
  // agree in summation order too
  a.chunk_tokens = hl_decode_chunk_tokens(ctx, batch, s->n_head_kv, max_ctx_h);
  a.max_chunks = (max_ctx_h + a.chunk_tokens - 1) / a.chunk_tokens;
  const size_t need = static_cast<size_t>(batch) * s->n_head * a.max_chunks;
  if (a.max_chunks > 65535 || need > kStaticTriples)
    return hl_fail(ctx, HL_ERR_CAPACITY,
                   "decode_static: batch %d x n_head %d x %d chunks = %zu partial slots, the static scratch holds %zu",
                   batch, s->n_head, a.max_chunks, need, kStaticTriples);
  a.q = hl::View{q->ptr, q->dtype, q->tok_stride, q->head_stride, q->dim_stride};
  a.out = hl::View{out->ptr, out->dtype, out->tok_stride, out->head_stride, out->dim_stride};
  a.gate = hl::View{nullptr, 0, 0, 0, 0};
  a.q_norm_w = s->q_norm_w;
  a.theta = ctx->theta_d;
  a.ctx_lens = ctx_lens;
  a.block_tables = block_tables;
  a.part_o = g_part_o_addr[ctx->device];
  a.part_ml = g_part_ml_addr[ctx->device];
  a.status = ctx->status_d;
  a.eps = s->rms_eps;
  a.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(s->head_dim));
  a.n_head = s->n_head;
  a.n_head_kv = s->n_head_kv;
  a.group = s->n_head / s->n_head_kv;
  a.rope_dim = s->rope_dim;
  a.rope_mode = s->rope_mode;
  a.block_tokens = kv->block_tokens;
  a.num_blocks = kv->num_blocks;
  a.max_blocks = max_blocks_per_seq;
  if (s->head_dim != 64 && s->head_dim != 128)
    return hl_fail(ctx, HL_ERR_UNSUPPORTED, "attn_decode_static: head_dim %d (the fixed scratch is laid out for 64 and 128)", s->head_dim);
  return s->head_dim == 64 ? launch<64>(ctx, kv, layer, a, batch) : launch<128>(ctx, kv, layer, a, batch);
}
