// Host side of libhl_b200: context, paged KV pool + TMA tensor maps, argument checks, launchers.
// The C ABI is declared in include/hl_b200.h.  No CPU fallback: every entry point either queues
// sm_100a kernels or returns an error status.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/hl_b200.h"
#include "attn_decode.cuh"
#include "attn_prefill_mma.cuh"
#include "attn_prefill_tc.cuh"
#include "attn_prefill_tc2.cuh"
#include "host_common.h"
#include "kv_append.cuh"
#include "linear_f16.cuh"
#include "linear_f16_pair.cuh"
#include "linear_gemv.cuh"
#include "linear_wide.cuh"

using namespace hl;

// ---------------------------------------------------------------------------------------------
// error plumbing
// ---------------------------------------------------------------------------------------------
int32_t hl_fail(hl_ctx* ctx, int32_t code, const char* fmt, ...) {
  if (ctx) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    ctx->err = buf;
  }
  return code;
}

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

int32_t hl_check_view(hl_ctx* ctx, const hl_view* v, const char* name) {
  if (!v || !v->ptr) return hl_fail(ctx, HL_ERR_ARG, "%s: null view or pointer", name);
  if (v->dtype != HL_DTYPE_F32 && v->dtype != HL_DTYPE_F16)
    return hl_fail(ctx, HL_ERR_ARG, "%s: dtype %d is neither f32 nor f16", name, v->dtype);
  const size_t el = v->dtype == HL_DTYPE_F16 ? 2 : 4;
  if (reinterpret_cast<uintptr_t>(v->ptr) % el)
    return hl_fail(ctx, HL_ERR_ALIGN, "%s: pointer not aligned to its element size", name);
  return HL_OK;
}

int32_t hl_check_shape(hl_ctx* ctx, const hl_kv* kv, const hl_attn_shape* s, int32_t layer) {
  if (!ctx) return HL_ERR_ARG;
  if (!kv || !s) return hl_fail(ctx, HL_ERR_ARG, "null kv or shape");
  if (layer < 0 || layer >= kv->n_layers)
    return hl_fail(ctx, HL_ERR_ARG, "layer %d outside [0, %d)", layer, kv->n_layers);
  if (s->n_head <= 0 || s->n_head_kv <= 0 || s->n_head % s->n_head_kv != 0)
    return hl_fail(ctx, HL_ERR_ARG, "GQA requires head_count divisible by head_count_kv");
  if (s->n_head_kv != kv->layer_kvh[layer] || s->head_dim != kv->head_dim)
    return hl_fail(ctx, HL_ERR_ARG, "shape (n_head_kv %d, head_dim %d) does not match layer %d of the KV pool (%d, %d)",
                   s->n_head_kv, s->head_dim, layer, kv->layer_kvh[layer], kv->head_dim);
  if (s->head_dim != 64 && s->head_dim != 128 && s->head_dim != 256)
    return hl_fail(ctx, HL_ERR_UNSUPPORTED, "head_dim %d: kernels are built for 64, 128 and 256", s->head_dim);
  if (s->rope_dim < 0 || s->rope_dim > s->head_dim || (s->rope_dim & 1))
    return hl_fail(ctx, HL_ERR_ARG, "rope_dim %d must be even and <= head_dim", s->rope_dim);
  if (s->rope_mode != HL_ROPE_INTERLEAVED && s->rope_mode != HL_ROPE_SPLIT_HALF)
    return hl_fail(ctx, HL_ERR_ARG, "rope_mode %d unknown", s->rope_mode);
  if (s->rope_dim > 0 && (!ctx->theta_d || ctx->theta_half < s->rope_dim / 2))
    return hl_fail(ctx, HL_ERR_ARG, "RoPE table not set or shorter than rope_dim/2 (hl_b200_set_rope)");
  return HL_OK;
}

namespace {
View to_view(const hl_view* v) { return View{v->ptr, v->dtype, v->tok_stride, v->head_stride, v->dim_stride}; }
inline int32_t check_view(hl_ctx* ctx, const hl_view* v, const char* name) { return hl_check_view(ctx, v, name); }
inline int32_t check_shape(hl_ctx* ctx, const hl_kv* kv, const hl_attn_shape* s, int32_t layer) {
  return hl_check_shape(ctx, kv, s, layer);
}
}  // namespace

int32_t hl_begin_timing(hl_ctx* ctx, float* gpu_ms) {
  if (gpu_ms) HL_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
  return HL_OK;
}
int32_t hl_end_timing(hl_ctx* ctx, float* gpu_ms) {
  HL_CUDA(ctx, cudaGetLastError());
  if (gpu_ms) {
    HL_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    HL_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
    HL_CUDA(ctx, cudaEventElapsedTime(gpu_ms, ctx->ev0, ctx->ev1));
  }
  return HL_OK;
}

// ---------------------------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------------------------
extern "C" int32_t hl_b200_create(int32_t device, void* stream, hl_ctx** out) {
  if (!out) return HL_ERR_ARG;
  *out = nullptr;
  int n_dev = 0;
  if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev) return HL_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return HL_ERR_CUDA;
  if (prop.major != 10) return HL_ERR_UNSUPPORTED;  // sm_100a cubins only; there is no other path
  if (cudaSetDevice(device) != cudaSuccess) return HL_ERR_CUDA;
  hl_ctx* ctx = new hl_ctx();
  ctx->device = device;
  ctx->n_sm = prop.multiProcessorCount;
  if (stream) {
    ctx->stream = static_cast<cudaStream_t>(stream);
  } else {
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
      delete ctx;
      return HL_ERR_CUDA;
    }
    ctx->own_stream = true;
  }
  bool ok = cudaEventCreate(&ctx->ev0) == cudaSuccess && cudaEventCreate(&ctx->ev1) == cudaSuccess &&
            cudaEventCreate(&ctx->ev2) == cudaSuccess && cudaEventCreate(&ctx->ev3) == cudaSuccess &&
            cudaMalloc(&ctx->status_d, 2 * sizeof(int32_t)) == cudaSuccess &&
            cudaMemset(ctx->status_d, 0, 2 * sizeof(int32_t)) == cudaSuccess;
  cudaDriverEntryPointQueryResult qres;
  void* fn = nullptr;
  ok = ok && cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
                 cudaSuccess &&
       fn != nullptr;
  if (!ok) {
    hl_b200_destroy(ctx);
    return HL_ERR_CUDA;
  }
  ctx->encode_tiled = fn;
  *out = ctx;
  return HL_OK;
}

extern "C" int32_t hl_b200_destroy(hl_ctx* ctx) {
  if (!ctx) return HL_ERR_ARG;
  cudaSetDevice(ctx->device);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  if (ctx->theta_d) cudaFree(ctx->theta_d);
  if (ctx->status_d) cudaFree(ctx->status_d);
  if (ctx->part_o) cudaFree(ctx->part_o);
  if (ctx->part_ml) cudaFree(ctx->part_ml);
  if (ctx->splitk_part) cudaFree(ctx->splitk_part);
  for (void* p : ctx->stage)
    if (p) cudaFree(p);
  if (ctx->cs_table) cudaFree(ctx->cs_table);
  if (ctx->ev0) cudaEventDestroy(ctx->ev0);
  if (ctx->ev1) cudaEventDestroy(ctx->ev1);
  if (ctx->ev2) cudaEventDestroy(ctx->ev2);
  if (ctx->ev3) cudaEventDestroy(ctx->ev3);
  for (int i = 0; i < 3; ++i) {
    if (ctx->side_done[i]) cudaEventDestroy(ctx->side_done[i]);
    if (ctx->side_stream[i]) cudaStreamDestroy(ctx->side_stream[i]);
  }
  if (ctx->fork_ev) cudaEventDestroy(ctx->fork_ev);
  if (ctx->own_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return HL_OK;
}

extern "C" const char* hl_b200_last_error(const hl_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

extern "C" int32_t hl_b200_sync(hl_ctx* ctx) {
  if (!ctx) return HL_ERR_ARG;
  HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return HL_OK;
}

extern "C" int32_t hl_b200_set_stream(hl_ctx* ctx, void* stream) {
  if (!ctx) return HL_ERR_ARG;
  if (ctx->own_stream) {
    cudaStreamSynchronize(ctx->stream);
    cudaStreamDestroy(ctx->stream);
    ctx->own_stream = false;
  }
  ctx->stream = static_cast<cudaStream_t>(stream);
  return HL_OK;
}

extern "C" int32_t hl_b200_device_status(hl_ctx* ctx, int32_t* code, int32_t* detail) {
  if (!ctx || !code) return HL_ERR_ARG;
  int32_t h[2] = {0, 0};
  HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  HL_CUDA(ctx, cudaMemcpy(h, ctx->status_d, sizeof h, cudaMemcpyDeviceToHost));
  if (h[0] != 0) HL_CUDA(ctx, cudaMemset(ctx->status_d, 0, sizeof h));
  *code = h[0];
  if (detail) *detail = h[1];
  if (h[0] != 0)
    hl_fail(ctx, h[0], "device status %d (detail %d): %s", h[0], h[1],
            h[0] == HL_ERR_TIMEOUT ? "a bounded wait gave up"
                                   : "block table entry or position outside the KV pool");
  return HL_OK;
}

extern "C" int64_t hl_b200_launch_count(const hl_ctx* ctx) { return ctx ? ctx->launches : -1; }

extern "C" int32_t hl_b200_set_tuning(hl_ctx* ctx, int32_t decode_chunk_tokens, int32_t prefill_kernel) {
  if (!ctx) return HL_ERR_ARG;
  if (decode_chunk_tokens < 0 || decode_chunk_tokens % 64 != 0)
    return hl_fail(ctx, HL_ERR_ARG, "decode_chunk_tokens must be 0 or a multiple of 64");
  if (prefill_kernel < 0 || prefill_kernel > 3) return hl_fail(ctx, HL_ERR_ARG, "prefill_kernel must be 0..3");
  ctx->decode_chunk = decode_chunk_tokens;
  ctx->prefill_kernel = prefill_kernel;
  return HL_OK;
}

// ---------------------------------------------------------------------------------------------
// bounded-wait self-test
// ---------------------------------------------------------------------------------------------
__global__ void selftest_timeout_kernel(int32_t* status, uint32_t max_polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);  // one arrival expected; none will ever come
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    bool ok = false;
    for (uint32_t i = 0; i < max_polls && !ok; ++i) ok = mbar_try_wait(&bar, 0);
    if (!ok) report(status, HL_ERR_TIMEOUT, 900);
  }
}

extern "C" int32_t hl_b200_selftest_wait_timeout(hl_ctx* ctx, int32_t max_polls) {
  if (!ctx) return HL_ERR_ARG;
  if (max_polls <= 0 || max_polls > (1 << 20)) return hl_fail(ctx, HL_ERR_ARG, "selftest: max_polls outside [1, 2^20]");
  HL_CUDA(ctx, cudaSetDevice(ctx->device));
  selftest_timeout_kernel<<<1, 32, 0, ctx->stream>>>(ctx->status_d, static_cast<uint32_t>(max_polls));
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  return HL_OK;
}

// ---------------------------------------------------------------------------------------------
// RoPE table
// ---------------------------------------------------------------------------------------------
extern "C" int32_t hl_b200_theta_table_h(float base, int32_t rope_dim, float* theta_h) {
  if (!theta_h || rope_dim <= 0 || (rope_dim & 1) || !(base > 0.f)) return HL_ERR_ARG;
  for (int i = 0; i < rope_dim / 2; ++i)
    theta_h[i] = powf(1.0f / base, (2.0f * static_cast<float>(i)) / static_cast<float>(rope_dim));
  return HL_OK;
}

extern "C" int32_t hl_b200_theta_llama3_scale_h(float* theta_h, int32_t half, float factor,
                                                float low_freq_factor, float high_freq_factor,
                                                int32_t original_ctx) {
  if (!theta_h || half <= 0 || !(factor > 0.f) || !(high_freq_factor > low_freq_factor) || original_ctx <= 0)
    return HL_ERR_ARG;
  const double two_pi = 6.283185307179586476925286766559;
  const double low_wavelen = static_cast<double>(original_ctx) / low_freq_factor;
  const double high_wavelen = static_cast<double>(original_ctx) / high_freq_factor;
  for (int i = 0; i < half; ++i) {
    const double th = theta_h[i];
    const double wavelen = two_pi / th;
    double r;
    if (wavelen < high_wavelen) {
      r = th;
    } else if (wavelen > low_wavelen) {
      r = th / factor;
    } else {
      const double smooth = (original_ctx / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor);
      r = (1.0 - smooth) * th / factor + smooth * th;
    }
    theta_h[i] = static_cast<float>(r);
  }
  return HL_OK;
}

extern "C" int32_t hl_b200_set_rope(hl_ctx* ctx, const float* theta_h, int32_t half) {
  if (!ctx) return HL_ERR_ARG;
  if (!theta_h || half <= 0 || half > 128) return hl_fail(ctx, HL_ERR_ARG, "set_rope: bad table");
  HL_CUDA(ctx, cudaSetDevice(ctx->device));
  HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->theta_half < half) {
    if (ctx->theta_d) cudaFree(ctx->theta_d);
    ctx->theta_d = nullptr;
    ctx->scratch_epoch++;
    HL_CUDA(ctx, cudaMalloc(&ctx->theta_d, half * sizeof(float)));
  }
  ctx->theta_half = half;
  ctx->cs_len = 0;  // the cos/sin table of the tcgen05 prefill is rebuilt from the new theta
  HL_CUDA(ctx, cudaMemcpy(ctx->theta_d, theta_h, half * sizeof(float), cudaMemcpyHostToDevice));
  return HL_OK;
}

// ---------------------------------------------------------------------------------------------
// KV pool
// ---------------------------------------------------------------------------------------------
static int32_t make_map(hl_ctx* ctx, CUtensorMap* map, void* pool, uint64_t rows, int head_dim, int box_rows) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(head_dim), rows};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(head_dim) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, pool, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return hl_fail(ctx, HL_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return HL_OK;
}

extern "C" int32_t hl_b200_kv_create(hl_ctx* ctx, int32_t n_layers, int32_t n_head_kv, int32_t head_dim,
                                     int32_t block_tokens, int32_t num_blocks, hl_kv** out) {
  return hl_b200_kv_create_layers(ctx, n_layers, nullptr, n_head_kv, head_dim, block_tokens, num_blocks, out);
}

extern "C" int32_t hl_b200_kv_create_layers(hl_ctx* ctx, int32_t n_layers, const int32_t* layer_n_head_kv,
                                            int32_t n_head_kv, int32_t head_dim, int32_t block_tokens,
                                            int32_t num_blocks, hl_kv** out) {
  if (!ctx) return HL_ERR_ARG;
  if (!out) return hl_fail(ctx, HL_ERR_ARG, "kv_create: null out");
  *out = nullptr;
  if (n_layers <= 0 || n_head_kv <= 0 || num_blocks <= 0) return hl_fail(ctx, HL_ERR_ARG, "kv_create: non-positive size");
  int max_kvh = n_head_kv;
  for (int l = 0; layer_n_head_kv && l < n_layers; ++l) {
    if (layer_n_head_kv[l] < 0) return hl_fail(ctx, HL_ERR_ARG, "kv_create: negative KV head count at layer %d", l);
    if (layer_n_head_kv[l] > max_kvh) max_kvh = layer_n_head_kv[l];
  }
  if (head_dim != 64 && head_dim != 128 && head_dim != 256)
    return hl_fail(ctx, HL_ERR_UNSUPPORTED, "kv_create: head_dim must be 64, 128 or 256");
  if (block_tokens <= 0 || block_tokens % 16 != 0) return hl_fail(ctx, HL_ERR_ARG, "kv_create: block_tokens must be a multiple of 16");
  if (static_cast<uint64_t>(num_blocks) * max_kvh * block_tokens >= (1ull << 31))
    return hl_fail(ctx, HL_ERR_CAPACITY, "kv_create: pool has too many rows for 32-bit TMA coordinates");
  HL_CUDA(ctx, cudaSetDevice(ctx->device));
  hl_kv* kv = new hl_kv();
  kv->n_layers = n_layers;
  kv->n_head_kv = n_head_kv;
  kv->head_dim = head_dim;
  kv->block_tokens = block_tokens;
  kv->num_blocks = num_blocks;
  kv->bytes_each = static_cast<uint64_t>(num_blocks) * n_head_kv * block_tokens * head_dim * 2;
  kv->layer_kvh.assign(n_layers, n_head_kv);
  kv->layer_bytes.assign(n_layers, 0);
  kv->k.assign(n_layers, nullptr);
  kv->v.assign(n_layers, nullptr);
  kv->k_map.resize(n_layers);
  kv->v_map.resize(n_layers);
  kv->k_map128.resize(n_layers);
  kv->v_map128.resize(n_layers);
  for (int l = 0; l < n_layers; ++l) {
    // a layer's own KV head count where one is given and positive, the default otherwise (naive.nim:3562-3563)
    if (layer_n_head_kv && layer_n_head_kv[l] > 0) kv->layer_kvh[l] = layer_n_head_kv[l];
    const uint64_t rows = static_cast<uint64_t>(num_blocks) * kv->layer_kvh[l] * block_tokens;
    const size_t bytes = rows * head_dim * 2;
    kv->layer_bytes[l] = bytes;
    // Zero-filled so that rows of a partly filled block always hold finite values.
    if (cudaMalloc(&kv->k[l], bytes) != cudaSuccess || cudaMalloc(&kv->v[l], bytes) != cudaSuccess ||
        cudaMemsetAsync(kv->k[l], 0, bytes, ctx->stream) != cudaSuccess ||
        cudaMemsetAsync(kv->v[l], 0, bytes, ctx->stream) != cudaSuccess) {
      cudaGetLastError();
      hl_b200_kv_destroy(ctx, kv);
      return hl_fail(ctx, HL_ERR_CUDA, "kv_create: out of device memory at layer %d (%zu bytes per pool)", l, bytes);
    }
    int32_t rc = make_map(ctx, &kv->k_map[l], kv->k[l], rows, head_dim, 16);
    if (rc == HL_OK) rc = make_map(ctx, &kv->v_map[l], kv->v[l], rows, head_dim, 16);
    // Wider boxes for the tcgen05 prefill kernel when a block holds a whole 128-key tile.
    const int wide = block_tokens >= 128 && block_tokens % 128 == 0 ? 128 : 16;
    if (rc == HL_OK) rc = make_map(ctx, &kv->k_map128[l], kv->k[l], rows, head_dim, wide);
    if (rc == HL_OK) rc = make_map(ctx, &kv->v_map128[l], kv->v[l], rows, head_dim, wide);
    if (rc != HL_OK) {
      hl_b200_kv_destroy(ctx, kv);
      return rc;
    }
  }
  HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  *out = kv;
  return HL_OK;
}

extern "C" int32_t hl_b200_kv_destroy(hl_ctx* ctx, hl_kv* kv) {
  if (!ctx || !kv) return HL_ERR_ARG;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  for (auto p : kv->k)
    if (p) cudaFree(p);
  for (auto p : kv->v)
    if (p) cudaFree(p);
  delete kv;
  return HL_OK;
}

extern "C" int32_t hl_b200_kv_layer(const hl_kv* kv, int32_t layer, void** k_pool, void** v_pool, size_t* bytes_each) {
  if (!kv || layer < 0 || layer >= kv->n_layers) return HL_ERR_ARG;
  if (k_pool) *k_pool = kv->k[layer];
  if (v_pool) *v_pool = kv->v[layer];
  if (bytes_each) *bytes_each = kv->layer_bytes[layer];
  return HL_OK;
}

// ---------------------------------------------------------------------------------------------
// append
// ---------------------------------------------------------------------------------------------
static int32_t launch_append(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s, const hl_view* k,
                             const hl_view* v, int32_t n_tok, int32_t start_pos, int32_t batch_mode,
                             const int32_t* ctx_lens, const int32_t* tables, int32_t max_blocks) {
  int32_t rc = check_shape(ctx, kv, s, layer);
  if (rc == HL_OK) rc = check_view(ctx, k, "k");
  if (rc == HL_OK) rc = check_view(ctx, v, "v");
  if (rc != HL_OK) return rc;
  if (n_tok <= 0) return hl_fail(ctx, HL_ERR_ARG, "append requires at least one token");
  if (!tables || max_blocks <= 0) return hl_fail(ctx, HL_ERR_ARG, "append: null or empty block table");
  if (batch_mode && !ctx_lens) return hl_fail(ctx, HL_ERR_ARG, "append: null ctx_lens");
  if (!batch_mode) {
    if (start_pos < 0) return hl_fail(ctx, HL_ERR_ARG, "append: negative start_pos");
    if (static_cast<int64_t>(start_pos) + n_tok > static_cast<int64_t>(max_blocks) * kv->block_tokens)
      return hl_fail(ctx, HL_ERR_CAPACITY, "append exceeds KV cache capacity (%d + %d > %lld)", start_pos, n_tok,
                     static_cast<long long>(max_blocks) * kv->block_tokens);
  }
  AppendArgs a{};
  a.k = to_view(k);
  a.v = to_view(v);
  a.k_pool = kv->k[layer];
  a.v_pool = kv->v[layer];
  a.k_norm_w = s->k_norm_w;
  a.theta = ctx->theta_d;
  a.ctx_lens = ctx_lens;
  a.block_tables = tables;
  a.status = ctx->status_d;
  a.eps = s->rms_eps;
  a.n_tok = n_tok;
  a.start_pos = start_pos;
  a.batch_mode = batch_mode;
  a.n_head_kv = s->n_head_kv;
  a.rope_dim = s->rope_dim;
  a.rope_mode = s->rope_mode;
  a.block_tokens = kv->block_tokens;
  a.num_blocks = kv->num_blocks;
  a.max_blocks = max_blocks;
  const int64_t rows = static_cast<int64_t>(n_tok) * s->n_head_kv;
  const unsigned grid = static_cast<unsigned>((rows + 3) / 4);
  HL_CUDA(ctx, cudaSetDevice(ctx->device));
  // the append may overlap the tail of the kernel in front, and the attention kernel behind (decode or prefill) starts
  // its set-up and query prologue during the append
  HL_CUDA(ctx, s->head_dim == 64    ? launch_pdl(kv_append_kernel<64>, dim3(grid), dim3(128), 0, ctx->stream, a)
               : s->head_dim == 128 ? launch_pdl(kv_append_kernel<128>, dim3(grid), dim3(128), 0, ctx->stream, a)
                                    : launch_pdl(kv_append_kernel<256>, dim3(grid), dim3(128), 0, ctx->stream, a));
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  return HL_OK;
}

extern "C" int32_t hl_b200_kv_append_seq(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                                         const hl_view* k, const hl_view* v, int32_t n_tok, int32_t start_pos,
                                         const int32_t* block_table, int32_t n_blocks_in_table) {
  return launch_append(ctx, kv, layer, shape, k, v, n_tok, start_pos, 0, nullptr, block_table, n_blocks_in_table);
}

extern "C" int32_t hl_b200_kv_append_batch(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                                           const hl_view* k, const hl_view* v, int32_t batch, const int32_t* ctx_lens,
                                           const int32_t* block_tables, int32_t max_blocks_per_seq) {
  return launch_append(ctx, kv, layer, shape, k, v, batch, 0, 1, ctx_lens, block_tables, max_blocks_per_seq);
}

// ---------------------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------------------
template <int HD>
static int32_t launch_decode(hl_ctx* ctx, hl_kv* kv, int32_t layer, const DecodeArgs& a, int32_t batch) {
  constexpr int NW = 4, STAGES = HD == 256 ? 2 : (HD == 128 ? 3 : 4);  // 64 KiB of K and V per stage at head_dim 256
  using Cfg = DecodeCfg<HD, NW, STAGES>;
  auto kern = attn_decode_kernel<HD, NW, STAGES>;
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    HL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured[ctx->device & 15] = true;
  }
  dim3 grid(a.max_chunks, a.n_head_kv, batch);
  HL_CUDA(ctx, launch_pdl(kern, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, ctx->stream, kv->k_map[layer], kv->v_map[layer], a));
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  if (a.max_chunks > 1) {
    HL_CUDA(ctx, launch_pdl(attn_combine_kernel<HD>, dim3(a.n_head, batch), dim3(HD), 0, ctx->stream, a));
    ctx->launches++;
    HL_CUDA(ctx, cudaGetLastError());
  }
  return HL_OK;
}

int32_t hl_decode_chunk_tokens(const hl_ctx* ctx, int32_t batch, int32_t n_head_kv, int32_t max_ctx) {
  if (ctx->decode_chunk > 0) return ctx->decode_chunk;
  // Aim at about eight CTAs per SM over the whole grid; never below two 64-token stages (a single short sequence
  // is latency-bound: fewer partials to merge beat more CTAs).
  const int64_t base = static_cast<int64_t>(batch) * n_head_kv;
  int64_t chunk = (static_cast<int64_t>(max_ctx) * base) / (8 * ctx->n_sm);
  chunk = ((chunk + 63) / 64) * 64;
  if (chunk < 128) chunk = 128;
  if (chunk > 1024) chunk = 1024;
  return static_cast<int32_t>(chunk);
}

int32_t hl_decode_reserve(hl_ctx* ctx, size_t need) {
  if (need <= ctx->part_cap) return HL_OK;  // grow-only scratch, like ensureActivationBuffers (naive.nim:241-262)
  HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->part_o) cudaFree(ctx->part_o);
  if (ctx->part_ml) cudaFree(ctx->part_ml);
  ctx->part_o = ctx->part_ml = nullptr;
  ctx->part_cap = 0;
  ctx->scratch_epoch++;
  HL_CUDA(ctx, cudaMalloc(&ctx->part_o, need * 128 * sizeof(float)));
  HL_CUDA(ctx, cudaMalloc(&ctx->part_ml, need * 2 * sizeof(float)));
  ctx->part_cap = need;
  return HL_OK;
}

static int32_t decode_impl(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s, const hl_view* q,
                           int32_t batch, const int32_t* ctx_lens, int32_t max_ctx_h, const int32_t* block_tables,
                           int32_t max_blocks_per_seq, const hl_view* gate, const hl_view* out, float* gpu_ms,
                           void* const* bcast = nullptr, int32_t n_bcast = 0) {
  int32_t rc = check_shape(ctx, kv, s, layer);
  if (rc == HL_OK) rc = check_view(ctx, q, "q");
  if (rc == HL_OK) rc = check_view(ctx, out, "out");
  if (rc == HL_OK && gate) rc = check_view(ctx, gate, "gate");
  if (rc != HL_OK) return rc;
  if (batch <= 0 || batch > 65535) return hl_fail(ctx, HL_ERR_ARG, "decode: batch %d outside [1, 65535]", batch);
  if (!ctx_lens || !block_tables || max_blocks_per_seq <= 0) return hl_fail(ctx, HL_ERR_ARG, "decode: null ctx_lens or block table");
  if (max_ctx_h <= 0) return hl_fail(ctx, HL_ERR_ARG, "decode: max_ctx_h must be positive");
  if (static_cast<int64_t>(max_ctx_h) > static_cast<int64_t>(max_blocks_per_seq) * kv->block_tokens)
    return hl_fail(ctx, HL_ERR_CAPACITY, "KV cache full: context %d exceeds the block table (%lld tokens)", max_ctx_h,
                   static_cast<long long>(max_blocks_per_seq) * kv->block_tokens);
  const int group = s->n_head / s->n_head_kv;
  if (group > 16) return hl_fail(ctx, HL_ERR_UNSUPPORTED, "decode: n_head / n_head_kv = %d > 16", group);
  HL_CUDA(ctx, cudaSetDevice(ctx->device));

  DecodeArgs a{};
  a.chunk_tokens = ctx->chunk_override > 0 ? ctx->chunk_override : hl_decode_chunk_tokens(ctx, batch, s->n_head_kv, max_ctx_h);
  a.max_chunks = (max_ctx_h + a.chunk_tokens - 1) / a.chunk_tokens;
  if (a.max_chunks > 65535) return hl_fail(ctx, HL_ERR_UNSUPPORTED, "decode: too many chunks");
  if (a.max_chunks > 1) {
    // slots of 128 floats: one per (sequence, head, chunk) up to head_dim 128, two at head_dim 256
    const size_t need = static_cast<size_t>(batch) * s->n_head * a.max_chunks * ((s->head_dim + 127) / 128);
    if (ctx->part_base + need > ctx->part_cap) {
      if (ctx->part_base != 0) return hl_fail(ctx, HL_ERR_CAPACITY, "decode: scratch of a batch slice was not reserved");
      rc = hl_decode_reserve(ctx, need);
      if (rc != HL_OK) return rc;
    }
  }
  a.q = to_view(q);
  a.out = to_view(out);
  a.gate = gate ? to_view(gate) : View{nullptr, 0, 0, 0, 0};
  a.q_norm_w = s->q_norm_w;
  a.theta = ctx->theta_d;
  a.ctx_lens = ctx_lens;
  a.block_tables = block_tables;
  a.part_o = ctx->part_o + ctx->part_base * 128;
  a.part_ml = ctx->part_ml + ctx->part_base * 2;
  a.status = ctx->status_d;
  a.eps = s->rms_eps;
  a.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(s->head_dim));
  a.n_head = s->n_head;
  a.n_head_kv = s->n_head_kv;
  a.group = group;
  a.rope_dim = s->rope_dim;
  a.rope_mode = s->rope_mode;
  a.block_tokens = kv->block_tokens;
  a.num_blocks = kv->num_blocks;
  a.max_blocks = max_blocks_per_seq;
  a.n_bcast = n_bcast;
  for (int i = 0; i < n_bcast; ++i) a.bcast[i] = bcast[i];
  a.early_q = ctx->chain_pdl ? 1 : 0;

  rc = hl_begin_timing(ctx, gpu_ms);
  if (rc != HL_OK) return rc;
  rc = s->head_dim == 64    ? launch_decode<64>(ctx, kv, layer, a, batch)
       : s->head_dim == 128 ? launch_decode<128>(ctx, kv, layer, a, batch)
                            : launch_decode<256>(ctx, kv, layer, a, batch);
  if (rc != HL_OK) return rc;
  return hl_end_timing(ctx, gpu_ms);
}

extern "C" int32_t hl_b200_attn_decode(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s,
                                       const hl_view* q, int32_t batch, const int32_t* ctx_lens, int32_t max_ctx_h,
                                       const int32_t* block_tables, int32_t max_blocks_per_seq, const hl_view* out,
                                       float* gpu_ms) {
  return decode_impl(ctx, kv, layer, s, q, batch, ctx_lens, max_ctx_h, block_tables, max_blocks_per_seq, nullptr, out,
                     gpu_ms);
}

extern "C" int32_t hl_b200_attn_decode_gated(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s,
                                             const hl_view* q, int32_t batch, const int32_t* ctx_lens,
                                             int32_t max_ctx_h, const int32_t* block_tables,
                                             int32_t max_blocks_per_seq, const hl_view* gate, const hl_view* out,
                                             float* gpu_ms) {
  if (ctx && !gate) return hl_fail(ctx, HL_ERR_ARG, "decode_gated: null gate view");
  return decode_impl(ctx, kv, layer, s, q, batch, ctx_lens, max_ctx_h, block_tables, max_blocks_per_seq, gate, out,
                     gpu_ms);
}

extern "C" int32_t hl_b200_attn_decode_bcast(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s,
                                             const hl_view* q, int32_t batch, const int32_t* ctx_lens,
                                             int32_t max_ctx_h, const int32_t* block_tables,
                                             int32_t max_blocks_per_seq, const hl_view* out,
                                             void* const* peer_out_ptrs, int32_t n_peers, float* gpu_ms) {
  if (!ctx) return HL_ERR_ARG;
  if (n_peers < 0 || n_peers > 7) return hl_fail(ctx, HL_ERR_ARG, "decode_bcast: n_peers %d outside [0, 7]", n_peers);
  if (n_peers > 0 && !peer_out_ptrs) return hl_fail(ctx, HL_ERR_ARG, "decode_bcast: null peer pointer list");
  const size_t el = out && out->dtype == HL_DTYPE_F16 ? 2 : 4;
  for (int i = 0; i < n_peers; ++i) {
    if (!peer_out_ptrs[i]) return hl_fail(ctx, HL_ERR_ARG, "decode_bcast: null peer pointer %d", i);
    if (reinterpret_cast<uintptr_t>(peer_out_ptrs[i]) % el)
      return hl_fail(ctx, HL_ERR_ALIGN, "decode_bcast: peer pointer %d not aligned to the output element size", i);
  }
  return decode_impl(ctx, kv, layer, s, q, batch, ctx_lens, max_ctx_h, block_tables, max_blocks_per_seq, nullptr, out,
                     gpu_ms, peer_out_ptrs, n_peers);
}

// ---------------------------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------------------------
template <int HD>
static int32_t launch_prefill_mma(hl_ctx* ctx, hl_kv* kv, int32_t layer, const PrefillArgs& a) {
  constexpr int NW = HD == 256 ? 4 : 8, STAGES = 2;  // head_dim 256: 64 query rows per CTA (registers: 128 accumulators per thread)
  using Cfg = PrefillMmaCfg<HD, NW, STAGES>;
  auto kern = attn_prefill_mma_kernel<HD, NW, STAGES>;
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    HL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured[ctx->device & 15] = true;
  }
  dim3 grid(a.n_head, (a.n_tok + Cfg::kBM - 1) / Cfg::kBM);
  kern<<<grid, (NW + 1) * 32, Cfg::kSmemBytes, ctx->stream>>>(kv->k_map[layer], kv->v_map[layer], a);
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  return HL_OK;
}

static int32_t prefill_impl(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s, const hl_view* q,
                            int32_t n_tok, int32_t start_pos, const int32_t* block_table, int32_t n_blocks_in_table,
                            const hl_view* out, void* const* bcast, int32_t n_bcast, float* gpu_ms,
                            const hl_view* gate = nullptr) {
  int32_t rc = check_shape(ctx, kv, s, layer);
  if (rc == HL_OK) rc = check_view(ctx, q, "q");
  if (rc == HL_OK) rc = check_view(ctx, out, "out");
  if (rc == HL_OK && gate) rc = check_view(ctx, gate, "gate");
  if (rc != HL_OK) return rc;
  if (n_tok <= 0) return hl_fail(ctx, HL_ERR_ARG, "prefill requires at least one token");
  if (start_pos < 0) return hl_fail(ctx, HL_ERR_ARG, "prefill: negative start_pos");
  if (!block_table || n_blocks_in_table <= 0) return hl_fail(ctx, HL_ERR_ARG, "prefill: null or empty block table");
  if (static_cast<int64_t>(start_pos) + n_tok > static_cast<int64_t>(n_blocks_in_table) * kv->block_tokens)
    return hl_fail(ctx, HL_ERR_CAPACITY, "prefill exceeds KV cache capacity (%d + %d > %lld)", start_pos, n_tok,
                   static_cast<long long>(n_blocks_in_table) * kv->block_tokens);
  if (s->n_head > 65535) return hl_fail(ctx, HL_ERR_UNSUPPORTED, "prefill: too many heads");
  if (n_tok > 65535 * 128) return hl_fail(ctx, HL_ERR_UNSUPPORTED, "prefill: more than 65535 query tiles in one call");
  HL_CUDA(ctx, cudaSetDevice(ctx->device));

  PrefillArgs a{};
  a.q = to_view(q);
  a.out = to_view(out);
  a.gate = gate ? to_view(gate) : View{nullptr, 0, 0, 0, 0};
  a.q_norm_w = s->q_norm_w;
  a.theta = ctx->theta_d;
  a.block_table = block_table;
  a.status = ctx->status_d;
  a.eps = s->rms_eps;
  a.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(s->head_dim));
  a.n_tok = n_tok;
  a.start_pos = start_pos;
  a.n_head = s->n_head;
  a.n_head_kv = s->n_head_kv;
  a.group = s->n_head / s->n_head_kv;
  a.rope_dim = s->rope_dim;
  a.rope_mode = s->rope_mode;
  a.block_tokens = kv->block_tokens;
  a.num_blocks = kv->num_blocks;
  a.n_blocks_in_table = n_blocks_in_table;

  rc = hl_begin_timing(ctx, gpu_ms);
  if (rc != HL_OK) return rc;
  const bool want_tc =
      n_bcast > 0 || ctx->prefill_kernel == 2 || (ctx->prefill_kernel == 0 && hl_prefill_tc_default(a, s->head_dim));
  if (ctx->prefill_kernel == 3) {
    if (!hl_prefill_tc2_supported(a, s->head_dim))
      return hl_fail(ctx, HL_ERR_UNSUPPORTED, "prefill: the two-SM tcgen05 kernel takes head_dim 128 only");
    rc = hl_launch_prefill_tc2(ctx, kv, layer, a, bcast, n_bcast);
  } else if (want_tc) {
    if (!hl_prefill_tc_supported(a, s->head_dim))
      return hl_fail(ctx, HL_ERR_UNSUPPORTED, "prefill: the tcgen05 kernel does not take this shape");
    rc = hl_launch_prefill_tc(ctx, kv, layer, a, s->head_dim, bcast, n_bcast);
  } else {
    rc = s->head_dim == 64    ? launch_prefill_mma<64>(ctx, kv, layer, a)
         : s->head_dim == 128 ? launch_prefill_mma<128>(ctx, kv, layer, a)
                              : launch_prefill_mma<256>(ctx, kv, layer, a);
  }
  if (rc != HL_OK) return rc;
  return hl_end_timing(ctx, gpu_ms);
}

extern "C" int32_t hl_b200_attn_prefill(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s,
                                        const hl_view* q, int32_t n_tok, int32_t start_pos, const int32_t* block_table,
                                        int32_t n_blocks_in_table, const hl_view* out, float* gpu_ms) {
  return prefill_impl(ctx, kv, layer, s, q, n_tok, start_pos, block_table, n_blocks_in_table, out, nullptr, 0, gpu_ms);
}

extern "C" int32_t hl_b200_attn_prefill_bcast(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s,
                                              const hl_view* q, int32_t n_tok, int32_t start_pos,
                                              const int32_t* block_table, int32_t n_blocks_in_table,
                                              const hl_view* out, void* const* peer_out_ptrs, int32_t n_peers,
                                              float* gpu_ms) {
  if (!ctx) return HL_ERR_ARG;
  if (n_peers < 0 || n_peers > 7) return hl_fail(ctx, HL_ERR_ARG, "prefill_bcast: n_peers %d outside [0, 7]", n_peers);
  if (n_peers > 0 && !peer_out_ptrs) return hl_fail(ctx, HL_ERR_ARG, "prefill_bcast: null peer pointer list");
  for (int i = 0; i < n_peers; ++i) {
    if (!peer_out_ptrs[i]) return hl_fail(ctx, HL_ERR_ARG, "prefill_bcast: null peer pointer %d", i);
    if (reinterpret_cast<uintptr_t>(peer_out_ptrs[i]) % 16 != 0 || (out && reinterpret_cast<uintptr_t>(out->ptr) % 16 != 0))
      return hl_fail(ctx, HL_ERR_ALIGN, "prefill_bcast: output pointers must be 16-byte aligned");
  }
  return prefill_impl(ctx, kv, layer, s, q, n_tok, start_pos, block_table, n_blocks_in_table, out, peer_out_ptrs,
                      n_peers, gpu_ms);
}

extern "C" int32_t hl_b200_attn_prefill_gated(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* s,
                                              const hl_view* q, int32_t n_tok, int32_t start_pos,
                                              const int32_t* block_table, int32_t n_blocks_in_table,
                                              const hl_view* gate, const hl_view* out, float* gpu_ms) {
  if (ctx && !gate) return hl_fail(ctx, HL_ERR_ARG, "prefill_gated: null gate view");
  return prefill_impl(ctx, kv, layer, s, q, n_tok, start_pos, block_table, n_blocks_in_table, out, nullptr, 0, gpu_ms,
                      gate);
}

// ---------------------------------------------------------------------------------------------
// dense fp16 projection: out = A . W^T (+ residual)
// ---------------------------------------------------------------------------------------------
static int32_t make_map_2d(hl_ctx* ctx, CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                           int box_rows) {
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return hl_fail(ctx, HL_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return HL_OK;
}

// Launch of the decode GEMV (M <= 4, K % 8 == 0, 16-byte aligned W rows).  g.a / x per mode as in GemvArgs.
static int32_t launch_gemv_fused(hl_ctx* ctx, GemvArgs p) {
  const LinearArgs& g = p.g;
  constexpr int R = 4;
  const int64_t groups = (g.N + R - 1) / R;
  int ks = 1;
  while (ks < 8 && groups * ks < static_cast<int64_t>(ctx->n_sm) * 12 && g.K / (ks * 2) >= 256) ks *= 2;
  p.ks = ks;
  p.kslice = ((g.K + ks - 1) / ks + 255) / 256 * 256;
  const size_t smem = static_cast<size_t>(g.M) * g.K * 2 + 8 * 4 * R * sizeof(float);
  if (smem > 200 * 1024) return hl_fail(ctx, HL_ERR_UNSUPPORTED, "decode projection: M * K too large for shared memory");
  const unsigned grid = static_cast<unsigned>((groups * ks + 7) / 8);
  auto kern = g.M == 1 ? linear_gemv_fused_kernel<1, R> : (g.M == 2 ? linear_gemv_fused_kernel<2, R> : linear_gemv_fused_kernel<4, R>);
  static bool configured[16][3] = {};
  bool& conf = configured[ctx->device & 15][g.M == 1 ? 0 : (g.M == 2 ? 1 : 2)];
  if (smem > 48 * 1024 && !conf) {
    HL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    conf = true;
  }
  // programmatic stream serialisation: the kernel may start while its predecessor drains; it prefetches weights,
  // then waits for the predecessor (griddepcontrol.wait) before it touches activations
  static const bool no_pdl = getenv("HL_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = no_pdl ? 0 : 1;
  HL_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  return HL_OK;
}

int32_t hl_linear_decode_fused(hl_ctx* ctx, int32_t mode, int32_t swiglu, const void* a, int64_t lda, const float* norm_w,
                               float eps, const void* w, int64_t ldw, void* out, int32_t out_dtype, int64_t ldo,
                               const float* resid, int64_t ldr, int32_t M, int32_t N, int32_t K) {
  if (!ctx) return HL_ERR_ARG;
  if (!a || !w || !out || (mode == kGemvRmsNorm && !norm_w)) return hl_fail(ctx, HL_ERR_ARG, "decode projection: null pointer");
  if (M <= 0 || M > 4 || N <= 0 || K <= 0 || (K & 7) || (ldw & 7) || ldw >= (1 << 28) || (reinterpret_cast<uintptr_t>(w) & 15))
    return hl_fail(ctx, HL_ERR_UNSUPPORTED, "decode projection: needs 1 <= M <= 4, K % 8 == 0 and 16-byte aligned weight rows");
  if (mode < kGemvPlain || mode > kGemvRmsNorm) return hl_fail(ctx, HL_ERR_ARG, "decode projection: bad prologue mode");
  if (swiglu && ((N & 1) || resid || out_dtype != HL_DTYPE_F16))
    return hl_fail(ctx, HL_ERR_ARG, "decode projection: the SwiGLU epilogue needs an even N, fp16 output and no residual");
  if (lda < K || ldw < K || ldo < (swiglu ? N / 2 : N) || (resid && ldr < N))
    return hl_fail(ctx, HL_ERR_ARG, "decode projection: leading dimension too small");
  HL_CUDA(ctx, cudaSetDevice(ctx->device));
  GemvArgs p{};
  p.g.a = mode == kGemvRmsNorm ? nullptr : static_cast<const __half*>(a);
  p.x = mode == kGemvRmsNorm ? static_cast<const float*>(a) : nullptr;
  p.ldx = lda;
  p.norm_w = norm_w;
  p.eps = eps;
  p.mode = mode;
  p.swiglu = swiglu;
  p.g.w = static_cast<const __half*>(w);
  p.g.out = out;
  p.g.resid = resid;
  p.g.lda = lda;
  p.g.ldw = ldw;
  p.g.ldo = ldo;
  p.g.ldr = ldr;
  p.g.M = M;
  p.g.N = N;
  p.g.K = K;
  p.g.out_dtype = out_dtype;
  p.g.status = ctx->status_d;
  return launch_gemv_fused(ctx, p);
}

// split-K scratch of the several-row projection (grow-only), and the launch of the reduction behind it
static int32_t ensure_splitk(hl_ctx* ctx, size_t floats) {
  if (floats <= ctx->splitk_cap) return HL_OK;
  HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->splitk_part) cudaFree(ctx->splitk_part);
  ctx->splitk_part = nullptr;
  ctx->splitk_cap = 0;
  ctx->scratch_epoch++;
  HL_CUDA(ctx, cudaMalloc(&ctx->splitk_part, floats * sizeof(float)));
  ctx->splitk_cap = floats;
  return HL_OK;
}
static int32_t launch_splitk_reduce(hl_ctx* ctx, const LinearArgs& g, int splits) {
  const int64_t quads = static_cast<int64_t>((g.N + 3) / 4) * g.M;
  static const bool no_pdl = getenv("HL_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((quads + 255) / 256));
  cfg.blockDim = dim3(256);
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = no_pdl ? 0 : 1;
  HL_CUDA(ctx, cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, static_cast<const float*>(ctx->splitk_part), splits, g));
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  return HL_OK;
}

static int32_t make_map_2d(hl_ctx* ctx, CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                           int box_rows);

// 2 <= M <= 128: tcgen05 with W on the M side of the MMA (linear_wide.cuh)
static int32_t launch_wide(hl_ctx* ctx, const LinearArgs& g) {
  using Cfg = LinearWideCfg;
  const int tiles_n = (g.N + Cfg::BW - 1) / Cfg::BW;
  int splits = 1;
  // as many splits as still fit one wave of two CTAs per SM (a second, partly filled wave costs more than it buys)
  while (static_cast<int64_t>(tiles_n) * splits * 2 <= 2 * ctx->n_sm && g.K / (splits * 2) >= 256) splits *= 2;
  const int kl = (((g.K + splits - 1) / splits) + 63) / 64 * 64;
  splits = (g.K + kl - 1) / kl;
  WideArgs p{};
  p.g = g;
  p.splits = splits;
  p.kl = kl;
  p.m_pad = (g.M + 15) / 16 * 16;
  if (splits > 1) {
    const int32_t rc = ensure_splitk(ctx, static_cast<size_t>(splits) * g.M * g.N);
    if (rc != HL_OK) return rc;
    p.part = ctx->splitk_part;
  }
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    HL_CUDA(ctx, cudaFuncSetAttribute(linear_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured[ctx->device & 15] = true;
  }
  CUtensorMap w_map, a_map;
  int32_t rc = make_map_2d(ctx, &w_map, g.w, g.N, g.K, g.ldw, Cfg::BW);
  if (rc == HL_OK) rc = make_map_2d(ctx, &a_map, g.a, g.M, g.K, g.lda, p.m_pad);
  if (rc != HL_OK) return rc;
  static const bool no_pdl = getenv("HL_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(tiles_n, splits);
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = no_pdl ? 0 : 1;
  HL_CUDA(ctx, cudaLaunchKernelEx(&cfg, linear_wide_kernel, w_map, a_map, p));
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  return splits > 1 ? launch_splitk_reduce(ctx, g, splits) : HL_OK;
}

extern "C" int32_t hl_b200_linear_f16(hl_ctx* ctx, const void* a, int64_t lda, const void* w, int64_t ldw, void* out,
                                      int32_t out_dtype, int64_t ldo, const float* resid, int64_t ldr, int32_t M,
                                      int32_t N, int32_t K, float* gpu_ms) {
  if (!ctx) return HL_ERR_ARG;
  if (!a || !w || !out) return hl_fail(ctx, HL_ERR_ARG, "linear: null pointer");
  if (M <= 0 || N <= 0 || K <= 0) return hl_fail(ctx, HL_ERR_ARG, "linear: non-positive size");
  if (out_dtype != HL_DTYPE_F32 && out_dtype != HL_DTYPE_F16) return hl_fail(ctx, HL_ERR_ARG, "linear: bad out dtype");
  return hl_linear_f16_impl(ctx, a, lda, w, ldw, out, out_dtype, ldo, resid, ldr, M, N, K, gpu_ms);
}

extern "C" int32_t hl_b200_linear_f16_silu(hl_ctx* ctx, const void* a, int64_t lda, const void* w, int64_t ldw, void* h,
                                           int64_t ldh, int32_t M, int32_t N, int32_t K, float* gpu_ms) {
  if (!ctx) return HL_ERR_ARG;
  if (!a || !w || !h) return hl_fail(ctx, HL_ERR_ARG, "linear: null pointer");
  if (M < 16 || N <= 0 || (N & 1) || K <= 0 || ldh < N / 2)
    return hl_fail(ctx, HL_ERR_ARG, "linear (silu): needs M >= 16, even N and ldh >= N / 2");
  return hl_linear_f16_impl(ctx, a, lda, w, ldw, h, hl::kLinearOutSiluPairs, N, nullptr, 0, M, N, K, gpu_ms, ldh);
}

int32_t hl_linear_f16_impl(hl_ctx* ctx, const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int32_t out_dtype,
                           int64_t ldo, const float* resid, int64_t ldr, int32_t M, int32_t N, int32_t K, float* gpu_ms,
                           int64_t ld_store) {
  if (out_dtype != HL_DTYPE_F32 && out_dtype != HL_DTYPE_F16 && out_dtype != hl::kLinearOutSiluPairs)
    return hl_fail(ctx, HL_ERR_ARG, "linear: bad out dtype");
  if (lda < K || ldw < K || ldo < N || (resid && ldr < N)) return hl_fail(ctx, HL_ERR_ARG, "linear: leading dimension too small");
  if (ld_store > 0) ldo = ld_store;  // the pair form stores N / 2 columns per row
  HL_CUDA(ctx, cudaSetDevice(ctx->device));
  LinearArgs g{};
  g.a = static_cast<const __half*>(a);
  g.w = static_cast<const __half*>(w);
  g.out = out;
  g.resid = resid;
  g.lda = lda;
  g.ldw = ldw;
  g.ldo = ldo;
  g.ldr = ldr;
  g.M = M;
  g.N = N;
  g.K = K;
  g.out_dtype = out_dtype;
  g.status = ctx->status_d;
  int32_t rc = hl_begin_timing(ctx, gpu_ms);
  if (rc != HL_OK) return rc;
  static const bool no_wide = getenv("HL_B200_NO_WIDE") != nullptr;
  const bool silu = out_dtype == hl::kLinearOutSiluPairs;  // implemented by the two tcgen05 GEMMs only (M >= 16)
  if (M >= 2 && M <= 128 && !no_wide && !silu && !(lda & 7) && !(ldw & 7) && !(reinterpret_cast<uintptr_t>(a) & 15) &&
      !(reinterpret_cast<uintptr_t>(w) & 15)) {
    rc = launch_wide(ctx, g);
    if (rc != HL_OK) return rc;
    return hl_end_timing(ctx, gpu_ms);
  }
  if (M <= 4 && !(K & 7) && !(ldw & 7) && ldw < (1 << 28) && !(reinterpret_cast<uintptr_t>(w) & 15) &&
      static_cast<size_t>(M) * K * 2 + 512 <= 200 * 1024) {
    GemvArgs p{};
    p.g = g;
    p.mode = kGemvPlain;
    rc = launch_gemv_fused(ctx, p);
    if (rc != HL_OK) return rc;
    return hl_end_timing(ctx, gpu_ms);
  }
  if (M < 16) {
    const unsigned grid = static_cast<unsigned>((static_cast<int64_t>(N) * 32 + 255) / 256);
    if (M <= 4)
      linear_gemv_kernel<4><<<grid, 256, 0, ctx->stream>>>(g);
    else
      linear_gemv_kernel<16><<<grid, 256, 0, ctx->stream>>>(g);
  } else {
    if ((lda & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
      return hl_fail(ctx, HL_ERR_ALIGN, "linear: A and W need 16-byte aligned bases and row strides (multiples of 8 halfs)");
    static const bool no_pair = getenv("HL_B200_GEMM_NO_PAIR") != nullptr;
    if (M >= 512 && (!no_pair || out_dtype == hl::kLinearOutSiluPairs)) {
      // 256 x 256 tiles on SM pairs (linear_f16_pair.cuh)
      using Cfg = LinearPairCfg;
      static bool configured2[16] = {};
      if (!configured2[ctx->device & 15]) {
        HL_CUDA(ctx, cudaFuncSetAttribute(linear_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        configured2[ctx->device & 15] = true;
      }
      CUtensorMap a_map, w_map;
      rc = make_map_2d(ctx, &a_map, a, M, K, lda, Cfg::BM);
      if (rc == HL_OK) rc = make_map_2d(ctx, &w_map, w, N, K, ldw, Cfg::BNH);
      if (rc != HL_OK) return rc;
      const int n_tiles = ((M + 255) / 256) * ((N + 255) / 256);
      const int max_pairs = ctx->n_sm / 2;
      const int pairs = n_tiles < max_pairs ? n_tiles : max_pairs;
      linear_gemm_pair_kernel<<<2 * pairs, Cfg::kThreads, Cfg::kSmemBytes, ctx->stream>>>(a_map, w_map, g);
    } else {
      using Cfg = LinearGemmCfg;
      static bool configured[16] = {};
      if (!configured[ctx->device & 15]) {
        HL_CUDA(ctx, cudaFuncSetAttribute(linear_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        configured[ctx->device & 15] = true;
      }
      CUtensorMap a_map, w_map;
      rc = make_map_2d(ctx, &a_map, a, M, K, lda, Cfg::BM);
      if (rc == HL_OK) rc = make_map_2d(ctx, &w_map, w, N, K, ldw, Cfg::BN);
      if (rc != HL_OK) return rc;
      const int n_tiles = ((M + Cfg::BM - 1) / Cfg::BM) * ((N + Cfg::BN - 1) / Cfg::BN);
      const int grid = n_tiles < ctx->n_sm ? n_tiles : ctx->n_sm;
      linear_gemm_kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, ctx->stream>>>(a_map, w_map, g);
    }
  }
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  return hl_end_timing(ctx, gpu_ms);
}
