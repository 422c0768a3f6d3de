/*
 * hl_backend -- the reference's backend contract, as a C ABI over the B200 attention path.
 *
 * hippo_leap selects a backend at compile time (src/hippo_leap/inference.nim:7-14) and calls
 * seven procs on it.  Each entry point below is the C side of one of them; the Nim module
 * src/hippo_leap/backends/b200.nim binds them with importc and keeps the Nim signatures.
 * Like the reference backends, the state is one model per process (module-level singletons,
 * src/hippo_leap/backends/naive.nim:235-239) and callers serialise their calls.
 *
 * The model behind this contract here is an ATTENTION-ONLY stand-in: the projection, FFN and
 * vocabulary layers of a real model are outside the hot path, so per layer the token id selects
 * a query / key / value row from seeded tables (in place of embedding + Q/K/V projections),
 * the layers' attention outputs are summed, and one [q_dim, n_vocab] matrix maps the sum to
 * logits.  Everything between those -- QK-norm, RoPE, KV append, causal GQA prefill, split-KV
 * decode -- is the product path, driven exactly as forwardPrefill / forwardDecode drive it.
 *
 * Status codes are hl_status (hl_b200.h); 0 = ok.  Nothing throws or aborts.
 */
#ifndef HL_BACKEND_H_
#define HL_BACKEND_H_

#include <stdint.h>

#include "hl_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The HParams fields that parameterise the path (src/hippo_leap/model.nim:24-50). */
typedef struct hl_hparams {
  int32_t n_vocab, n_layer, n_head, n_head_kv, head_dim, rope_dim;
  float rope_freq_base, rms_eps;
  int32_t rope_mode;      /* HL_ROPE_SPLIT_HALF for the drop-in (what the reference GPU path does) */
  int32_t llama3_scaling; /* non-zero: apply the llama3 frequency scaling to the theta table */
} hl_hparams;

/* Host float32 weights of the stand-in model. */
typedef struct hl_standin_weights {
  const float* eq;     /* [n_layer][n_vocab][n_head * head_dim]     token -> query row */
  const float* ek;     /* [n_layer][n_vocab][n_head_kv * head_dim]  token -> key row   */
  const float* ev;     /* [n_layer][n_vocab][n_head_kv * head_dim]  token -> value row */
  const float* wout;   /* [n_head * head_dim][n_vocab]                                  */
  const float* q_norm; /* [n_layer][head_dim] or NULL (attn_q_norm.weight)              */
  const float* k_norm; /* [n_layer][head_dim] or NULL (attn_k_norm.weight)              */
} hl_standin_weights;

/* The KvCache fields the contract reads and writes (src/hippo_leap/backend_types.nim:41-49).
 * Callers may reset cur_len to 0 between requests (src/hippo_leap/inference.nim:58). */
typedef struct hl_kv_cache {
  int32_t cur_len, max_len, n_head_kv, head_dim;
  void* gpu_cache; /* hl_kv*: the paged pool; GpuKvCache.k/v[layer] come from hl_b200_kv_layer */
} hl_kv_cache;

/* initKvCache(hp, maxLen): src/hippo_leap/backends/naive.nim:3912-3931. */
int32_t hl_backend_init_kv_cache(int32_t device, const hl_hparams* hp, int32_t max_len, hl_kv_cache* out);
int32_t hl_backend_free_kv_cache(hl_kv_cache* cache);
/* loadModelBackend(m, hp): naive.nim:3956-3958 (weight upload + theta table, naive.nim:3850-3861). */
int32_t hl_backend_load_model(int32_t device, const hl_hparams* hp, const hl_standin_weights* w);
/* unloadModelBackend(): naive.nim:3960-3962. */
int32_t hl_backend_unload_model(void);
/* forwardPrefill(m, tokens, cache) -> logits of the LAST position, [1, n_vocab] like the
 * megakernel backend (megakernel.nim:2498); argmaxLast accepts that shape (sampling.nim:20-31).
 * Like the reference it always starts at position 0 and leaves cache.cur_len = n
 * (naive.nim:4075-4076, 4586-4587).  Errors as naive.nim:3969-3976: empty prompt, prompt longer
 * than the cache. */
int32_t hl_backend_forward_prefill(const int32_t* tokens_h, int32_t n, hl_kv_cache* cache, float* logits_h);
/* Chunked prefill / prefix reuse -- no counterpart in the reference, whose forwardPrefill always restarts at
 * position 0 (naive.nim:3125; the wish is in docs/v2.5.md:40-47).  The n tokens take positions cache.cur_len ..
 * cache.cur_len + n - 1 on top of whatever the cache already holds up to cur_len; cur_len += n; logits of the last
 * of them.  A long prompt can be fed in pieces, and a caller that resets cur_len to the length of a shared prefix
 * re-uses that prefix's keys and values. */
int32_t hl_backend_forward_prefill_chunk(const int32_t* tokens_h, int32_t n, hl_kv_cache* cache, float* logits_h);
/* forwardDecode(m, token, cache): naive.nim:4592-5100.  pos = cache.cur_len; "KV cache full"
 * when pos >= max_len (naive.nim:4598-4599). */
int32_t hl_backend_forward_decode(int32_t token, hl_kv_cache* cache, float* logits_h);
/* forwardDecodeToken(m, token, cache): naive.nim:5102-5546 (argmax on the device, 4-byte download). */
int32_t hl_backend_forward_decode_token(int32_t token, hl_kv_cache* cache, int32_t* next_token);
/* forwardDecodeTokenTimed(m, token, cache, gpuMs): megakernel.nim:2514-2529. */
int32_t hl_backend_forward_decode_token_timed(int32_t token, hl_kv_cache* cache, int32_t* next_token,
                                              float* gpu_ms);
/* forwardDecodeToken[Timed] replay one captured CUDA graph per token by default (the counterpart of the
 * megakernel backend's graph mode, -d:useGraphCapture, megakernel.nim:2458-2479); 0 switches to plain
 * launches.  Results are identical either way. */
int32_t hl_backend_set_decode_graph(int32_t enabled);
const char* hl_backend_last_error(void);
/* Kernel launches issued by the backend's context so far. */
int64_t hl_backend_launch_count(void);

/* ---- the same contract on a DENSE llama / qwen3 model ------------------------------------------
 * The first step beyond the hot path: the layers either side of attention for the reference's
 * lkAttentionFfn layer kind (naive.nim:4054-4086, 4656-4771) with dense fp16 weights -- embedding,
 * RMSNorm, Q/K/V and output projections, SwiGLU FFN, final norm, vocabulary projection, argmax -- so
 * that forwardPrefill / forwardDecode run a whole model forward on the GPU.  Weights are plain host
 * arrays (row-major [out][in] fp16 matrices, fp32 norm vectors): there is no GGUF reader and none of the
 * reference's quantised formats here. */
typedef struct hl_dense_hparams {
  int32_t n_vocab, n_emb, n_layer, n_ffn, n_head, n_head_kv, head_dim, rope_dim;
  float rope_freq_base, rms_eps;
  int32_t rope_mode, llama3_scaling;
} hl_dense_hparams;

typedef struct hl_dense_weights {
  const uint16_t* tok_emb;   /* [n_vocab][n_emb] fp16                            token_embd.weight   */
  const float* attn_norm;    /* [n_layer][n_emb]                                 blk.N.attn_norm     */
  const uint16_t* wq;        /* [n_layer][n_head*head_dim][n_emb]                blk.N.attn_q        */
  const uint16_t* wk;        /* [n_layer][n_head_kv*head_dim][n_emb]             blk.N.attn_k        */
  const uint16_t* wv;        /* [n_layer][n_head_kv*head_dim][n_emb]             blk.N.attn_v        */
  const uint16_t* wo;        /* [n_layer][n_emb][n_head*head_dim]                blk.N.attn_output   */
  const float* q_norm;       /* [n_layer][head_dim] or NULL                      blk.N.attn_q_norm   */
  const float* k_norm;       /* [n_layer][head_dim] or NULL                      blk.N.attn_k_norm   */
  const float* ffn_norm;     /* [n_layer][n_emb]                                 blk.N.ffn_norm      */
  const uint16_t* w_gate;    /* [n_layer][n_ffn][n_emb]                          blk.N.ffn_gate      */
  const uint16_t* w_up;      /* [n_layer][n_ffn][n_emb]                          blk.N.ffn_up        */
  const uint16_t* w_down;    /* [n_layer][n_emb][n_ffn]                          blk.N.ffn_down      */
  const float* out_norm;     /* [n_emb]                                          output_norm         */
  const uint16_t* w_out;     /* [n_vocab][n_emb]                                 output              */
} hl_dense_weights;

int32_t hl_dense_init_kv_cache(int32_t device, const hl_dense_hparams* hp, int32_t max_len, hl_kv_cache* out);
int32_t hl_dense_free_kv_cache(hl_kv_cache* cache);
int32_t hl_dense_load_model(int32_t device, const hl_dense_hparams* hp, const hl_dense_weights* w);
int32_t hl_dense_unload_model(void);
/* forwardPrefill: logits of the last position [n_vocab]; starts at position 0, sets cur_len = n. */
int32_t hl_dense_forward_prefill(const int32_t* tokens_h, int32_t n, hl_kv_cache* cache, float* logits_h);
/* Chunked prefill / prefix reuse on the dense model: as hl_backend_forward_prefill_chunk. */
int32_t hl_dense_forward_prefill_chunk(const int32_t* tokens_h, int32_t n, hl_kv_cache* cache, float* logits_h);
/* forwardDecode: one token at position cache.cur_len; "KV cache full" at capacity. */
int32_t hl_dense_forward_decode(int32_t token, hl_kv_cache* cache, float* logits_h);
/* forwardDecodeTokenTimed: argmax on the device, optional device time of the step. */
int32_t hl_dense_forward_decode_token_timed(int32_t token, hl_kv_cache* cache, int32_t* next_token, float* gpu_ms);
/* ---- several sequences decoded together (continuous-batching hook) ------------------------------------------------
 * No counterpart in the reference, which holds ONE sequence per process (inference.nim:28; the wish for batched
 * serving is in docs/v3.5.md:24-35).  A batch owns one shared page pool for max_seqs sequences of up to max_len
 * tokens; each decode step takes any subset of them, reads every weight once for all of their tokens, and runs the
 * attention path over their separate block tables.  Needs a loaded model (hl_dense_load_model); destroy batches
 * before unloading it. */
typedef struct hl_dense_batch hl_dense_batch;
int32_t hl_dense_batch_create(int32_t max_seqs, int32_t max_len, hl_dense_batch** out);
int32_t hl_dense_batch_destroy(hl_dense_batch* b);
/* Tokens held by sequence `seq`, or -1. */
int32_t hl_dense_batch_seq_len(const hl_dense_batch* b, int32_t seq);
/* Prefill of one sequence: n tokens at positions start_pos .. (0 starts it over; up to its current length continues
 * or re-uses a prefix); logits of the last of them [n_vocab]. */
int32_t hl_dense_batch_prefill(hl_dense_batch* b, int32_t seq, const int32_t* tokens_h, int32_t n, int32_t start_pos,
                               float* logits_h);
/* One decode step: token tokens_h[i] is appended to sequence seq_ids_h[i] (distinct), i < n_active.  Outputs, either
 * may be NULL: next_tokens_h[n_active] (argmax, first maximal index) and logits_h[n_active][n_vocab]. */
int32_t hl_dense_batch_decode(hl_dense_batch* b, const int32_t* seq_ids_h, const int32_t* tokens_h, int32_t n_active,
                              int32_t* next_tokens_h, float* logits_h, float* gpu_ms);

/* Decode steps replay one captured CUDA graph per token (default on); 0 queues the kernels one by one instead.
 * Same results either way.  The reference's megakernel backend replays a HIP graph per token the same way
 * (src/hippo_leap/backends/megakernel.nim:2458-2479). */
int32_t hl_dense_set_decode_graph(int32_t enabled);
const char* hl_dense_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* HL_BACKEND_H_ */
