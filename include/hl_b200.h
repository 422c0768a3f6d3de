/*
 * libhl_b200 -- C ABI of the B200 (sm_100a) attention hot path for hippo_leap.
 *
 * This is the boundary a `-d:backendB200` build of hippo_leap binds with `importc`
 * (src/hippo_leap/backends/b200.nim): RoPE (+ optional per-head QK RMSNorm), KV-cache
 * append, causal grouped-query attention for prefill and single-token attention over the
 * KV cache for decode.  Plain pointers and sizes only; no C++ or torch types.
 *
 * Conventions
 *  - Every entry point returns an hl_status (0 = ok).  Nothing throws, aborts or exits.
 *    hl_b200_last_error(ctx) gives the text of the last failure on that context.
 *  - Pointers are DEVICE pointers unless the name ends in _h (host).
 *  - Work is queued on the context's stream and NOT synchronised unless `gpu_ms` is
 *    non-NULL (then the call brackets its kernels with events, synchronises, and returns
 *    the device time in milliseconds) or hl_b200_sync() is called.
 *  - A context is not re-entrant: one thread at a time per context (the reference
 *    serialises callers with InferenceContext.lock, src/hippo_leap/inference.nim:53-54).
 *  - No CPU fallback exists.  Without a usable sm_100 device hl_b200_create fails.
 */
#ifndef HL_B200_H_
#define HL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum hl_status {
  HL_OK = 0,
  HL_ERR_ARG = 1,         /* null / negative / inconsistent argument            */
  HL_ERR_CAPACITY = 2,    /* position or block index beyond the KV pool         */
  HL_ERR_ALIGN = 3,       /* pointer or stride breaks an alignment rule         */
  HL_ERR_CUDA = 4,        /* a CUDA runtime / driver call failed                */
  HL_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up                 */
  HL_ERR_BOUNDS = 6,      /* a device-side index check failed (block table)     */
  HL_ERR_UNSUPPORTED = 7  /* shape outside what the kernels are built for       */
} hl_status;

enum { HL_DTYPE_F32 = 0, HL_DTYPE_F16 = 1 };

/* RoPE pairing.  INTERLEAVED rotates (2i, 2i+1) like the CPU op
 * (src/hippo_leap/tensor.nim:156-166); SPLIT_HALF rotates (i, i+ropeDim/2) like every
 * reference GPU kernel (src/hippo_leap/backends/naive.nim:3025-3030), which is what the
 * drop-in backend must use for an unchanged greedy token stream. */
enum { HL_ROPE_INTERLEAVED = 0, HL_ROPE_SPLIT_HALF = 1 };

typedef struct hl_ctx hl_ctx; /* one per process and device: stream, theta table, scratch */
typedef struct hl_kv hl_kv;   /* paged fp16 KV pool for all layers of one model          */

/* Shape of the attention op; the fields come from HParams (src/hippo_leap/model.nim:24-50). */
typedef struct hl_attn_shape {
  int32_t n_head;      /* query heads                                       */
  int32_t n_head_kv;   /* KV heads; n_head % n_head_kv == 0                 */
  int32_t head_dim;    /* 64, 128 or 256 (256: warp-MMA prefill, no static entry) */
  int32_t rope_dim;    /* even, <= head_dim; dims >= rope_dim not rotated   */
  int32_t rope_mode;   /* HL_ROPE_*                                         */
  float rms_eps;       /* eps of the QK RMSNorm (hp.rmsEps)                 */
  const float* q_norm_w; /* device [head_dim] or NULL: attn_q_norm.weight   */
  const float* k_norm_w; /* device [head_dim] or NULL: attn_k_norm.weight   */
} hl_attn_shape;

/* Strided view of a [n_tok][heads][head_dim] activation.  Strides are in ELEMENTS.
 * The reference's `[dim, S]` buffers (element (r, t) at r*S + t,
 * src/hippo_leap/backends/naive.nim:2984-2990) are {tok 1, head head_dim*S, dim S};
 * token-major buffers are {tok heads*head_dim, head head_dim, dim 1}. */
typedef struct hl_view {
  void* ptr;
  int32_t dtype; /* HL_DTYPE_* */
  int64_t tok_stride, head_stride, dim_stride;
} hl_view;

/* ---- context ---------------------------------------------------------------------- */

/* Replaces ensureGpuContext (src/hippo_leap/backends/naive.nim:237-262): binds `device`,
 * checks it is compute capability 10.x, adopts `stream` (a cudaStream_t) or creates one
 * when `stream` is NULL. */
int32_t hl_b200_create(int32_t device, void* stream, hl_ctx** out);
/* Replaces unloadModelBackend (naive.nim:3960-3962): frees everything the context owns. */
int32_t hl_b200_destroy(hl_ctx* ctx);
const char* hl_b200_last_error(const hl_ctx* ctx);
int32_t hl_b200_sync(hl_ctx* ctx);
/* Adopt another stream (e.g. the caller framework's current stream).  Here NULL means the
 * legacy default stream (handle 0), not "create one". */
int32_t hl_b200_set_stream(hl_ctx* ctx, void* stream);
/* Reads and clears the device status word that bounded waits and block-table checks set. */
int32_t hl_b200_device_status(hl_ctx* ctx, int32_t* code, int32_t* detail);
/* Number of kernels this context has launched since creation (for launch accounting). */
int64_t hl_b200_launch_count(const hl_ctx* ctx);

/* ---- RoPE table ------------------------------------------------------------------- */

/* Host helper: theta_i = powf(1/base, 2i/rope_dim), i < rope_dim/2 -- the table
 * ensureModelGpuPtrs builds (naive.nim:3850-3855). */
int32_t hl_b200_theta_table_h(float base, int32_t rope_dim, float* theta_h);
/* Host helper: the published "llama3" frequency scaling applied in place to a theta table
 * (no counterpart in the reference; a host-side transform of the table). */
int32_t hl_b200_theta_llama3_scale_h(float* theta_h, int32_t half, float factor,
                                     float low_freq_factor, float high_freq_factor,
                                     int32_t original_ctx);
/* Uploads theta[half] (replaces the upload at naive.nim:3856-3861). */
int32_t hl_b200_set_rope(hl_ctx* ctx, const float* theta_h, int32_t half);

/* ---- KV cache ---------------------------------------------------------------------
 * Replaces initGpuKvCache (naive.nim:3552-3567).  Per layer one K pool and one V pool,
 * fp16, laid out [num_blocks][n_head_kv][block_tokens][head_dim]: a (block, kv-head) tile is
 * one contiguous run of block_tokens rows of head_dim*2 bytes (128 or 256 B, so every row is
 * 128-byte aligned).  K is stored after QK-norm and RoPE, V raw, as in the reference.
 * block_tokens must be a multiple of 16.  A block table maps a sequence's logical block
 * (position / block_tokens) to a physical block: int32 [n_seq][max_blocks_per_seq]. */
int32_t hl_b200_kv_create(hl_ctx* ctx, int32_t n_layers, int32_t n_head_kv, int32_t head_dim,
                          int32_t block_tokens, int32_t num_blocks, hl_kv** out);
/* The same with a KV head count per layer, the layerNHeadKv argument of initGpuKvCache
 * (naive.nim:3552-3567; hybrid models whose attention layers differ): layer l holds
 * layer_n_head_kv[l] KV heads where that entry is positive, n_head_kv otherwise (the rule of
 * naive.nim:3562-3563); a null array means n_head_kv everywhere.  Every call that names a layer
 * checks its shape against that layer's count. */
int32_t hl_b200_kv_create_layers(hl_ctx* ctx, int32_t n_layers, const int32_t* layer_n_head_kv,
                                 int32_t n_head_kv, int32_t head_dim, int32_t block_tokens,
                                 int32_t num_blocks, hl_kv** out);
int32_t hl_b200_kv_destroy(hl_ctx* ctx, hl_kv* kv);
/* Device pointers and size in bytes of one layer's pools (to fill GpuKvCache.k/v[layer],
 * src/hippo_leap/backend_types.nim:28-34). */
int32_t hl_b200_kv_layer(const hl_kv* kv, int32_t layer, void** k_pool, void** v_pool,
                         size_t* bytes_each);

/* Replaces gpuQkNormPrefill(K) + gpuRopeAtPos(K) + gpuStoreKV(K), gpuStoreKV(V)
 * (naive.nim:4070-4076) for ONE sequence: n_tok tokens at positions start_pos.. of the
 * sequence whose block table (device, int32[n_blocks_in_table]) is given. */
int32_t hl_b200_kv_append_seq(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                              const hl_view* k, const hl_view* v, int32_t n_tok,
                              int32_t start_pos, const int32_t* block_table,
                              int32_t n_blocks_in_table);
/* Replaces gpuQkNorm(K) + the K half of gpuRopeQKDecode + gpuStoreKVPair, or
 * gpuFusedRopeStoreKV (naive.nim:4699-4710, 5186-5190) for a BATCH of sequences: token i
 * belongs to sequence i and is stored at position ctx_lens[i] - 1. */
int32_t hl_b200_kv_append_batch(hl_ctx* ctx, hl_kv* kv, int32_t layer,
                                const hl_attn_shape* shape, const hl_view* k, const hl_view* v,
                                int32_t batch, const int32_t* ctx_lens,
                                const int32_t* block_tables, int32_t max_blocks_per_seq);

/* ---- attention --------------------------------------------------------------------- */

/* Replaces gpuQkNormPrefill(Q) + gpuRopeAtPos(Q) + gpuAttentionPrefill
 * (naive.nim:4067-4078): for query token t (position start_pos + t) and head h,
 * out[t,h,:] = softmax_j((q.k_j)/sqrt(head_dim)) . v_j over keys j <= start_pos + t of KV
 * head h / (n_head / n_head_kv).  Q is normed, rotated and scaled inside the kernel; K/V
 * are read from the paged cache (append them first).  out: fp32 or fp16 view.
 * No 4096-key cap (naive.nim:3404) and start_pos may be non-zero. */
int32_t hl_b200_attn_prefill(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                             const hl_view* q, int32_t n_tok, int32_t start_pos,
                             const int32_t* block_table, int32_t n_blocks_in_table,
                             const hl_view* out, float* gpu_ms);

/* No counterpart in the reference (which has no multi-GPU code).  hl_b200_attn_prefill whose kernel
 * ALSO stores every output tile to up to 7 more destinations with the layout of `out`: the same
 * buffer on peer GPUs, mapped into this GPU's address space (CUDA IPC / symmetric memory).  With KV
 * heads sharded across GPUs, each GPU passes as `out` its own head slice of the full
 * [n_head][n_tok][head_dim] buffer and as peers the same slice of every other GPU's buffer: the
 * all-gather of head outputs then happens inside the attention kernel, tile by tile over NVLink,
 * instead of as a collective after it.  Peers must be synchronised by the caller before they read
 * (a barrier after the call's stream work has completed on every rank). */
int32_t hl_b200_attn_prefill_bcast(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                                   const hl_view* q, int32_t n_tok, int32_t start_pos,
                                   const int32_t* block_table, int32_t n_blocks_in_table,
                                   const hl_view* out, void* const* peer_out_ptrs, int32_t n_peers,
                                   float* gpu_ms);

/* Replaces gpuQkNorm(Q) + the Q half of gpuRopeQKDecode + gpuAttentionDecode
 * (naive.nim:4697-4717): one query token per sequence, sequence i attending its first
 * ctx_lens[i] cached keys (the new token's own K/V included: curLen = pos + 1).
 * Split-KV: the context is cut into chunks that run in parallel and a second pass merges
 * the partial (max, sum, out) triples.  max_ctx_h >= max_i ctx_lens[i] (host value, sizes
 * the grid and the scratch).  A device-side ctx_lens[i] beyond max_ctx_h rounded up to whole
 * chunks, or <= 0, sets the device status word to HL_ERR_BOUNDS (detail = i); the context is
 * clamped to the grid (resp. the output row zeroed) and nothing is read out of range. */
int32_t hl_b200_attn_decode(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                            const hl_view* q, int32_t batch, const int32_t* ctx_lens,
                            int32_t max_ctx_h, const int32_t* block_tables,
                            int32_t max_blocks_per_seq, const hl_view* out, float* gpu_ms);

/* No counterpart in the reference (which has no multi-GPU code).  hl_b200_attn_decode whose kernels ALSO store
 * every output row to up to 7 more destinations with the layout of `out`: the same buffer on peer GPUs, mapped
 * into this GPU's address space.  With KV heads sharded across GPUs (each GPU holds its KV heads of every
 * sequence's pages and runs the decode step on the query heads that map onto them), each GPU passes as `out` its
 * own head slice of the full [n_head][batch][head_dim] buffer and as peers the same slice of every other GPU's
 * buffer: the single all-gather of per-head outputs that replaces N copies of gpuAttentionDecode
 * (naive.nim:4714-4717) then happens inside the decode step's own stores.  Peers must be synchronised by the
 * caller before they read (a barrier after the call's stream work has completed on every rank). */
int32_t hl_b200_attn_decode_bcast(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                                  const hl_view* q, int32_t batch, const int32_t* ctx_lens,
                                  int32_t max_ctx_h, const int32_t* block_tables,
                                  int32_t max_blocks_per_seq, const hl_view* out,
                                  void* const* peer_out_ptrs, int32_t n_peers, float* gpu_ms);

/* The two attention calls with the output gate of the qwen3.5-MoE attention layers fused into
 * their epilogue: out <- sigmoid(gate) * out, replacing gpuAttnGate (naive.nim:2287-2300, applied at
 * naive.nim:4259-4260).  `gate` is indexed like `out` ([n_tok][n_head][head_dim] view).  The reference
 * de-interleaves a fused Q|gate projection first (gpuDeinterleaveQGatePrefill, naive.nim:2427-2456);
 * with strided views that copy is unnecessary: q = {ptr, head_stride 2*head_dim*S, ...} and
 * gate = {ptr + head_dim*S, same strides} address the fused buffer directly. */
int32_t hl_b200_attn_prefill_gated(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                                   const hl_view* q, int32_t n_tok, int32_t start_pos,
                                   const int32_t* block_table, int32_t n_blocks_in_table,
                                   const hl_view* gate, const hl_view* out, float* gpu_ms);
int32_t hl_b200_attn_decode_gated(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                                  const hl_view* q, int32_t batch, const int32_t* ctx_lens,
                                  int32_t max_ctx_h, const int32_t* block_tables,
                                  int32_t max_blocks_per_seq, const hl_view* gate, const hl_view* out,
                                  float* gpu_ms);

/* No counterpart in the reference.  hl_b200_attn_decode without any allocation, for callers that have
 * given all device memory to their own pool or cannot take the device-wide synchronisation of
 * cudaMalloc / cudaFree inside the decode loop.  Same arguments and result as hl_b200_attn_decode
 * (no gpu_ms); the split-KV partials live in a fixed 16.25 MiB array inside the library image, held
 * by every GPU that loads the library until the process exits.  Limit: batch * n_head * chunks <=
 * 32768 partial slots (chunks = ceil(max_ctx_h / chunk_tokens), 128..1024 tokens per chunk unless tuned); beyond it
 * the call returns HL_ERR_CAPACITY and launches nothing.  All calls on one GPU share the array: calls
 * whose kernels overlap on the GPU race, so serialise them.  The first call on each device resolves
 * the array's device address and configures the kernel; make it before any stream capture starts. */
int32_t hl_b200_attn_decode_static(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                                   const hl_view* q, int32_t batch, const int32_t* ctx_lens,
                                   int32_t max_ctx_h, const int32_t* block_tables,
                                   int32_t max_blocks_per_seq, const hl_view* out);

/* ---- host-buffer forms ------------------------------------------------------------------
 * The same two steps for callers whose activations live in HOST memory (float32, token-major
 * contiguous: q [n][n_head][head_dim], k and v [n][n_head_kv][head_dim], out like q).  Each call
 * copies its inputs to the device, runs append + attention, copies the result back and
 * synchronises -- the shape of one reference forward call, which uploads its inputs and
 * downloads its result around the kernels (naive.nim:4013, 4581-4584).  gpu_ms (optional)
 * receives the device time of the whole step, copies included. */
int32_t hl_b200_prefill_host(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl_attn_shape* shape,
                             const float* q_h, const float* k_h, const float* v_h, int32_t n_tok,
                             int32_t start_pos, const int32_t* block_table,
                             int32_t n_blocks_in_table, float* out_h, float* gpu_ms);
int32_t hl_b200_decode_step_host(hl_ctx* ctx, hl_kv* kv, int32_t layer,
                                 const hl_attn_shape* shape, const float* q_h, const float* k_h,
                                 const float* v_h, int32_t batch, const int32_t* ctx_lens,
                                 int32_t max_ctx_h, const int32_t* block_tables,
                                 int32_t max_blocks_per_seq, float* out_h, float* gpu_ms);

/* ---- projections either side of attention -------------------------------------------------
 * out[M, N] = A[M, K] . W[N, K]^T (+ residual[M, N]), fp16 A and W (row-major, leading dimensions in
 * elements), fp32 accumulation, fp32 or fp16 out.  Replaces gpuLinearCol for dense weights
 * (naive.nim:3466-3547: out[row, t] = sum_k W[row, k] x[k, t]); the residual add replaces the gpuAdd
 * that follows the output and down projections (naive.nim:4080, 4086).  M >= 16 runs a tcgen05 GEMM,
 * smaller M a weight-bandwidth-bound GEMV.  This is the first piece of the layers around the hot
 * path; the quantised GEMV family of the reference (naive.nim:354-1917) is not reproduced. */
int32_t hl_b200_linear_f16(hl_ctx* ctx, const void* a, int64_t lda, const void* w, int64_t ldw, void* out,
                           int32_t out_dtype, int64_t ldo, const float* resid, int64_t ldr, int32_t M,
                           int32_t N, int32_t K, float* gpu_ms);

/* The merged gate|up projection of a SwiGLU feed-forward block with its activation in the GEMM epilogue:
 * W [N, K] holds the gate and up rows INTERLEAVED (row 2c = gate row c, row 2c + 1 = up row c), and
 * h[M, N / 2] = fp16( silu(fp16 gate) * fp16 up ), silu(g) = g / (1 + expf(-g)) -- bit for bit what
 * hl_b200_linear_f16 with fp16 output followed by the reference's siluMulKernel (naive.nim:2179-2197,
 * call site naive.nim:4083-4085) gives, without the fp16 [M, N] intermediate.  M >= 16 (the tcgen05
 * GEMMs; the single-token decode path fuses the same activation into its GEMV). */
int32_t hl_b200_linear_f16_silu(hl_ctx* ctx, const void* a, int64_t lda, const void* w, int64_t ldw, void* h,
                                int64_t ldh, int32_t M, int32_t N, int32_t K, float* gpu_ms);

/* No counterpart in the reference.  Self-test of the bounded-wait machinery: launches one CTA that
 * waits, for at most `max_polls` polls, on a barrier nothing ever signals.  The wait gives up,
 * the kernel returns normally, and hl_b200_device_status then reports {HL_ERR_TIMEOUT, 900}.  The
 * context stays usable.  (How a lost signal would surface in the attention kernels, without one.) */
int32_t hl_b200_selftest_wait_timeout(hl_ctx* ctx, int32_t max_polls);

/* Tunables (0 = automatic): tokens per split-KV chunk for decode; which prefill kernel
 * runs (0 auto, 1 = warp-MMA kernel, 2 = tcgen05 kernel, 3 = tcgen05 kernel on SM pairs, head_dim 128). */
int32_t hl_b200_set_tuning(hl_ctx* ctx, int32_t decode_chunk_tokens, int32_t prefill_kernel);

#ifdef __cplusplus
}
#endif
#endif /* HL_B200_H_ */
