// Host-buffer forms of the two attention steps (declared in include/hl_b200.h).
#include <cuda_runtime.h>
#include <stdlib.h>

#include "../../include/hl_b200.h"
#include "host_common.h"

namespace {

int32_t ensure_stage(hl_ctx* ctx, int i, size_t bytes) {
  if (bytes <= ctx->stage_cap[i]) return HL_OK;
  HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->stage[i]) cudaFree(ctx->stage[i]);
  ctx->stage[i] = nullptr;
  ctx->stage_cap[i] = 0;
  ctx->scratch_epoch++;
  HL_CUDA(ctx, cudaMalloc(&ctx->stage[i], bytes));
  ctx->stage_cap[i] = bytes;
  return HL_OK;
}

hl_view dense_view(void* p, int heads, int hd) {
  return hl_view{p, HL_DTYPE_F32, static_cast<int64_t>(heads) * hd, hd, 1};
}

struct StepIo {
  hl_view q, k, v, out;
  size_t q_bytes, kv_bytes;
};

int32_t stage_in(hl_ctx* ctx, const hl_attn_shape* s, const float* q_h, const float* k_h, const float* v_h,
                 int32_t n, float* out_h, StepIo* io) {
  if (!ctx) return HL_ERR_ARG;
  if (!s || !q_h || !k_h || !v_h || !out_h) return hl_fail(ctx, HL_ERR_ARG, "host step: null argument");
  if (n <= 0 || s->n_head <= 0 || s->n_head_kv <= 0 || s->head_dim <= 0)
    return hl_fail(ctx, HL_ERR_ARG, "host step: non-positive size");
  HL_CUDA(ctx, cudaSetDevice(ctx->device));
  io->q_bytes = static_cast<size_t>(n) * s->n_head * s->head_dim * sizeof(float);
  io->kv_bytes = static_cast<size_t>(n) * s->n_head_kv * s->head_dim * sizeof(float);
  int32_t rc = ensure_stage(ctx, 0, io->q_bytes);
  if (rc == HL_OK) rc = ensure_stage(ctx, 1, io->kv_bytes);
  if (rc == HL_OK) rc = ensure_stage(ctx, 2, io->kv_bytes);
  if (rc == HL_OK) rc = ensure_stage(ctx, 3, io->q_bytes);
  if (rc != HL_OK) return rc;
  io->q = dense_view(ctx->stage[0], s->n_head, s->head_dim);
  io->k = dense_view(ctx->stage[1], s->n_head_kv, s->head_dim);
  io->v = dense_view(ctx->stage[2], s->n_head_kv, s->head_dim);
  io->out = dense_view(ctx->stage[3], s->n_head, s->head_dim);
  return HL_OK;
}

// Device-side address of a page-locked, mapped host buffer (cudaHostAlloc / cudaHostRegister memory under unified
// addressing), or nullptr for pageable memory.  The kernels can read and write such a buffer in place over PCIe.
void* mapped_host(const void* h) {
  cudaPointerAttributes at{};
  if (cudaPointerGetAttributes(&at, h) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer) return at.devicePointer;
  cudaGetLastError();
  return nullptr;
}

// Which buffers of a decode step are used in place when they are page-locked: bit 0 the output rows (the final
// stores become posted PCIe writes), bit 1 the new K / V rows (read once by the append kernel), bit 2 the query
// rows (read once by the decode prologue, spread over the kernel's run time instead of a copy in front of it).
// Measured on config 4: 0.262 ms per step with staged copies, 0.231-0.246 ms with all three in place.
// HL_B200_ZEROCOPY overrides the mask.
int zero_copy_mask() {
  static const int mask = [] {
    const char* e = getenv("HL_B200_ZEROCOPY");
    return e ? atoi(e) : 7;
  }();
  return mask;
}

}  // namespace

extern "C" int32_t hl_b200_prefill_host(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                                        const float* q_h, const float* k_h, const float* v_h, int32_t n_tok,
                                        int32_t start_pos, const int32_t* block_table, int32_t n_blocks_in_table,
                                        float* out_h, float* gpu_ms) {
  StepIo io;
  int32_t rc = stage_in(ctx, shape, q_h, k_h, v_h, n_tok, out_h, &io);
  if (rc != HL_OK) return rc;
  if (gpu_ms) HL_CUDA(ctx, cudaEventRecord(ctx->ev2, ctx->stream));
  HL_CUDA(ctx, cudaMemcpyAsync(io.q.ptr, q_h, io.q_bytes, cudaMemcpyHostToDevice, ctx->stream));
  HL_CUDA(ctx, cudaMemcpyAsync(io.k.ptr, k_h, io.kv_bytes, cudaMemcpyHostToDevice, ctx->stream));
  HL_CUDA(ctx, cudaMemcpyAsync(io.v.ptr, v_h, io.kv_bytes, cudaMemcpyHostToDevice, ctx->stream));
  rc = hl_b200_kv_append_seq(ctx, kv, layer, shape, &io.k, &io.v, n_tok, start_pos, block_table, n_blocks_in_table);
  if (rc == HL_OK)
    rc = hl_b200_attn_prefill(ctx, kv, layer, shape, &io.q, n_tok, start_pos, block_table, n_blocks_in_table, &io.out,
                              nullptr);
  if (rc != HL_OK) return rc;
  HL_CUDA(ctx, cudaMemcpyAsync(out_h, io.out.ptr, io.q_bytes, cudaMemcpyDeviceToHost, ctx->stream));
  if (gpu_ms) HL_CUDA(ctx, cudaEventRecord(ctx->ev3, ctx->stream));
  HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (gpu_ms) HL_CUDA(ctx, cudaEventElapsedTime(gpu_ms, ctx->ev2, ctx->ev3));
  return HL_OK;
}

// How many slices of the batch run as concurrent chains (append -> decode -> combine, each on a stream of its own) when
// all three inputs and the output are used in place: the new rows and queries of one slice cross PCIe while another
// slice computes, and the output rows -- written by the combine pass at the very end of a chain -- leave in several
// short bursts instead of one 2 MB burst behind the last kernel.  HL_B200_HOST_CHAINS overrides (1 = one chain).
static int host_chains(int32_t batch) {
  static const int forced = [] {
    const char* e = getenv("HL_B200_HOST_CHAINS");
    return e ? atoi(e) : 0;
  }();
  int n = forced > 0 ? forced : (batch >= 32 ? 4 : 1);
  if (n > 4) n = 4;
  if (n > batch) n = batch;
  return n < 1 ? 1 : n;
}

static int32_t ensure_side_streams(hl_ctx* ctx, int n_side) {
  if (!ctx->fork_ev) HL_CUDA(ctx, cudaEventCreateWithFlags(&ctx->fork_ev, cudaEventDisableTiming));
  for (int i = 0; i < n_side; ++i) {
    if (!ctx->side_stream[i]) HL_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->side_stream[i], cudaStreamNonBlocking));
    if (!ctx->side_done[i]) HL_CUDA(ctx, cudaEventCreateWithFlags(&ctx->side_done[i], cudaEventDisableTiming));
  }
  return HL_OK;
}

static hl_view rows_from(const hl_view& v, int64_t row) {
  hl_view o = v;
  o.ptr = static_cast<char*>(v.ptr) + row * v.tok_stride * (v.dtype == HL_DTYPE_F16 ? 2 : 4);
  return o;
}

extern "C" int32_t hl_b200_decode_step_host(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                                            const float* q_h, const float* k_h, const float* v_h, int32_t batch,
                                            const int32_t* ctx_lens, int32_t max_ctx_h, const int32_t* block_tables,
                                            int32_t max_blocks_per_seq, float* out_h, float* gpu_ms) {
  StepIo io;
  int32_t rc = stage_in(ctx, shape, q_h, k_h, v_h, batch, out_h, &io);
  if (rc != HL_OK) return rc;
  const int zc = zero_copy_mask();
  void* out_m = (zc & 1) ? mapped_host(out_h) : nullptr;
  void* k_m = (zc & 2) ? mapped_host(k_h) : nullptr;
  void* v_m = (zc & 2) ? mapped_host(v_h) : nullptr;
  void* q_m = (zc & 4) ? mapped_host(q_h) : nullptr;
  if (gpu_ms) HL_CUDA(ctx, cudaEventRecord(ctx->ev2, ctx->stream));
  if (q_m)
    io.q.ptr = q_m;
  else
    HL_CUDA(ctx, cudaMemcpyAsync(io.q.ptr, q_h, io.q_bytes, cudaMemcpyHostToDevice, ctx->stream));
  if (k_m && v_m) {
    io.k.ptr = k_m;
    io.v.ptr = v_m;
  } else {
    HL_CUDA(ctx, cudaMemcpyAsync(io.k.ptr, k_h, io.kv_bytes, cudaMemcpyHostToDevice, ctx->stream));
    HL_CUDA(ctx, cudaMemcpyAsync(io.v.ptr, v_h, io.kv_bytes, cudaMemcpyHostToDevice, ctx->stream));
  }
  if (out_m) io.out.ptr = out_m;
  const int chains = (q_m && k_m && v_m && out_m && max_ctx_h > 0 && shape->n_head_kv > 0) ? host_chains(batch) : 1;
  if (chains <= 1) {
    rc = hl_b200_kv_append_batch(ctx, kv, layer, shape, &io.k, &io.v, batch, ctx_lens, block_tables, max_blocks_per_seq);
    if (rc == HL_OK)
      rc = hl_b200_attn_decode(ctx, kv, layer, shape, &io.q, batch, ctx_lens, max_ctx_h, block_tables,
                               max_blocks_per_seq, &io.out, nullptr);
    if (rc != HL_OK) return rc;
  } else {
    // The chunk length of the WHOLE batch for every slice, so that each row is summed in the order the one-chain form
    // sums it (the two agree bit for bit); the partials scratch sized for the whole batch before anything runs.
    const int32_t chunk = hl_decode_chunk_tokens(ctx, batch, shape->n_head_kv, max_ctx_h);
    const int64_t max_chunks = (static_cast<int64_t>(max_ctx_h) + chunk - 1) / chunk;
    const size_t slots_per_seq = static_cast<size_t>(shape->n_head) * max_chunks * ((shape->head_dim + 127) / 128);
    if (max_chunks > 1) {
      rc = hl_decode_reserve(ctx, slots_per_seq * batch);
      if (rc != HL_OK) return rc;
    }
    rc = ensure_side_streams(ctx, chains - 1);
    if (rc != HL_OK) return rc;
    cudaStream_t main_stream = ctx->stream;
    HL_CUDA(ctx, cudaEventRecord(ctx->fork_ev, main_stream));  // the chains start behind whatever the stream holds
    const hl_view vq = io.q, vk = io.k, vv = io.v, vo = io.out;
    for (int c = 0; c < chains && rc == HL_OK; ++c) {
      const int32_t b0 = static_cast<int32_t>(static_cast<int64_t>(batch) * c / chains);
      const int32_t b1 = static_cast<int32_t>(static_cast<int64_t>(batch) * (c + 1) / chains);
      if (b1 <= b0) continue;
      cudaStream_t st = c == 0 ? main_stream : ctx->side_stream[c - 1];
      if (c > 0 && cudaStreamWaitEvent(st, ctx->fork_ev, 0) != cudaSuccess) rc = HL_ERR_CUDA;
      ctx->stream = st;
      ctx->part_base = max_chunks > 1 ? slots_per_seq * b0 : 0;
      ctx->chunk_override = chunk;
      const hl_view sq = rows_from(vq, b0), sk = rows_from(vk, b0), sv = rows_from(vv, b0), so = rows_from(vo, b0);
      const int32_t* lens = ctx_lens + b0;
      const int32_t* tabs = block_tables + static_cast<int64_t>(b0) * max_blocks_per_seq;
      if (rc == HL_OK) rc = hl_b200_kv_append_batch(ctx, kv, layer, shape, &sk, &sv, b1 - b0, lens, tabs, max_blocks_per_seq);
      if (rc == HL_OK)
        rc = hl_b200_attn_decode(ctx, kv, layer, shape, &sq, b1 - b0, lens, max_ctx_h, tabs, max_blocks_per_seq, &so, nullptr);
      if (c > 0) {
        if (cudaEventRecord(ctx->side_done[c - 1], st) != cudaSuccess ||
            cudaStreamWaitEvent(main_stream, ctx->side_done[c - 1], 0) != cudaSuccess)
          rc = rc == HL_OK ? HL_ERR_CUDA : rc;
      }
    }
    ctx->stream = main_stream;
    ctx->part_base = 0;
    ctx->chunk_override = 0;
    if (rc != HL_OK) {
      cudaStreamSynchronize(main_stream);
      for (int i = 0; i < chains - 1; ++i) cudaStreamSynchronize(ctx->side_stream[i]);
      return rc == HL_ERR_CUDA ? hl_fail(ctx, HL_ERR_CUDA, "decode_step_host: stream or event call failed") : rc;
    }
  }
  if (!out_m) HL_CUDA(ctx, cudaMemcpyAsync(out_h, io.out.ptr, io.q_bytes, cudaMemcpyDeviceToHost, ctx->stream));
  if (gpu_ms) HL_CUDA(ctx, cudaEventRecord(ctx->ev3, ctx->stream));
  HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (gpu_ms) HL_CUDA(ctx, cudaEventElapsedTime(gpu_ms, ctx->ev2, ctx->ev3));
  return HL_OK;
}
