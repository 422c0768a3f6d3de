/*
 * CPU float32 oracle for the attention hot path of hippo_leap.  TEST INFRASTRUCTURE ONLY:
 * nothing in the product library links, loads or calls this file.  It exists so that the
 * CUDA kernels can be checked against the reference's arithmetic.
 *
 * PARITY UNPINNED: the reference (a Nim program) cannot be built where this oracle is
 * developed, and its test-suite holds no golden vector for tensor.nim or for attention
 * (the only numeric pin, tests/integration_inference.nim:15-18, needs a GGUF model file
 * and the whole model stack).  What pins this file is a line-by-line reading of
 * src/hippo_leap/tensor.nim, cited per function below, plus an independent float64
 * cross-check in the test-suite.
 *
 * Part 1 restates the four tensor.nim primitives the path is built from, loop for loop:
 *   hl_ref_matmul            tensor.nim:63-81
 *   hl_ref_rmsnorm           tensor.nim:83-100
 *   hl_ref_softmax_last_dim  tensor.nim:120-139
 *   hl_ref_rope_inplace      tensor.nim:141-166   (interleaved pairs, theta by pow per element)
 * Nim's float32 pow/exp/cos/sin/sqrt lower to libm powf/expf/cosf/sinf/sqrtf; so do these.
 *
 * Part 2 is glue that tensor.nim does not have and that is therefore OURS, following the
 * order of operations of the reference GPU backend:
 *   theta table                  backends/naive.nim:3850-3855
 *   split-half RoPE pairing      backends/naive.nim:3025-3030
 *   QK-norm -> RoPE -> KV store -> attention    backends/naive.nim:4067-4078, 4697-4717
 *   kvh = h div (nHead div nHeadKv)             backends/naive.nim:3307-3308
 *   score = dot * (1/sqrt(headDim)) after the sum   backends/naive.nim:3328, 3415
 *   causal: query at position p attends keys 0..p   backends/naive.nim:3402
 *   optional sigmoid output gate                    backends/naive.nim:2287-2293
 * Attention rows are composed ONLY from the part-1 primitives (matmul for q.K^T and P.V,
 * softmax_last_dim for the row), so that every float32 rounding happens where tensor.nim
 * would put it.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ part 1: tensor.nim */

/* (m x k) * (k x n) -> (m x n), float32 accumulator, k innermost.  tensor.nim:63-81 */
void hl_ref_matmul(const float* a, const float* b, float* c, int m, int k, int n) {
  for (int i = 0; i < m; ++i) {
    const long arow = (long)i * k;
    const long crow = (long)i * n;
    for (int j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (int p = 0; p < k; ++p) acc += a[arow + p] * b[(long)p * n + j];
      c[crow + j] = acc;
    }
  }
}

/* RMS-normalise the last dimension and apply a per-dim weight.  tensor.nim:83-100 */
void hl_ref_rmsnorm(const float* x, const float* weight, float* out, long outer, int dim,
                    float eps) {
  for (long o = 0; o < outer; ++o) {
    float ss = 0.0f;
    const long base = o * dim;
    for (int i = 0; i < dim; ++i) {
      const float v = x[base + i];
      ss += v * v;
    }
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int i = 0; i < dim; ++i) out[base + i] = x[base + i] * inv * weight[i];
  }
}

/* softmax over the last dimension: max-subtract, exp, multiply by 1/sum.  tensor.nim:120-139 */
void hl_ref_softmax_last_dim(const float* x, float* out, long outer, int dim) {
  for (long o = 0; o < outer; ++o) {
    const long base = o * dim;
    float maxv = x[base];
    for (int i = 1; i < dim; ++i) maxv = fmaxf(maxv, x[base + i]);
    float sum = 0.0f;
    for (int i = 0; i < dim; ++i) {
      const float v = expf(x[base + i] - maxv);
      out[base + i] = v;
      sum += v;
    }
    const float inv = 1.0f / sum;
    for (int i = 0; i < dim; ++i) out[base + i] *= inv;
  }
}

/* RoPE in place on shape [outer, seqLen, dim]: pairs (2i, 2i+1), theta_i = pow(1/base, 2i/dim),
 * angle = float32(startPos + p) * theta_i.  tensor.nim:141-166 */
void hl_ref_rope_inplace(float* x, long outer, int seq_len, int dim, float base, int start_pos) {
  const float inv_base = 1.0f / base;
  for (long o = 0; o < outer; ++o) {
    const long outer_base = o * seq_len * (long)dim;
    for (int p = 0; p < seq_len; ++p) {
      const float pos = (float)(start_pos + p);
      const long row = outer_base + (long)p * dim;
      for (int i = 0; i < dim / 2; ++i) {
        const long idx0 = row + 2 * i;
        const long idx1 = row + 2 * i + 1;
        const float theta = powf(inv_base, (float)(2 * i) / (float)dim);
        const float angle = pos * theta;
        const float c = cosf(angle);
        const float s = sinf(angle);
        const float v0 = x[idx0];
        const float v1 = x[idx1];
        x[idx0] = v0 * c - v1 * s;
        x[idx1] = v0 * s + v1 * c;
      }
    }
  }
}

/* ------------------------------------------------------------------ part 2: glue (ours) */

enum { HL_REF_ROPE_INTERLEAVED = 0, HL_REF_ROPE_SPLIT_HALF = 1 };

/* theta_i = pow(1/base, 2i/ropeDim), i < ropeDim/2, float32 on the host.
 * backends/naive.nim:3850-3855 (same value as tensor.nim:158). */
void hl_ref_theta_table(float* theta, int rope_dim, float base) {
  const int half = rope_dim / 2;
  for (int i = 0; i < half; ++i)
    theta[i] = powf(1.0f / base, (2.0f * (float)i) / (float)rope_dim);
}

/* Rotate one head row x[0..head_dim) at integer position pos with a given theta table.
 * mode 0: pairs (2i, 2i+1) as tensor.nim:156-166; mode 1: pairs (i, i+half) as
 * backends/naive.nim:3025-3030.  Dims >= rope_dim are left alone (naive.nim:3200-3201). */
void hl_ref_rope_row(float* x, int rope_dim, const float* theta, int pos, int mode) {
  const int half = rope_dim / 2;
  const float fpos = (float)pos;
  for (int i = 0; i < half; ++i) {
    const int i0 = mode == HL_REF_ROPE_INTERLEAVED ? 2 * i : i;
    const int i1 = mode == HL_REF_ROPE_INTERLEAVED ? 2 * i + 1 : i + half;
    const float angle = fpos * theta[i];
    const float c = cosf(angle);
    const float s = sinf(angle);
    const float v0 = x[i0];
    const float v1 = x[i1];
    x[i0] = v0 * c - v1 * s;
    x[i1] = v0 * s + v1 * c;
  }
}

/* float32 -> IEEE half, round-to-nearest-even -> float32.  (The KV cache of the CUDA path
 * is fp16; the reference's own floatToHalf, quant.nim:98-107, truncates and is a weight
 * codec, so it is deliberately not what is restated here.) */
float hl_ref_round_fp16(float v) { return (float)(_Float16)v; }

/* One attention row from tensor.nim primitives.
 * q: [hd] (already normed + rotated); kc/vc: cache [*, n_head_kv, hd] token-major;
 * n_keys = pos + 1 keys are attended.  scratch: 2*n_keys + n_keys*hd floats. */
static void attention_row(const float* q, const float* kc, const float* vc, int kvh,
                          int n_head_kv, int hd, int n_keys, float* out, float* scratch) {
  float* kt = scratch;                      /* K^T slice [hd, n_keys]  (transpose: glue) */
  float* scores = kt + (long)hd * n_keys;   /* [1, n_keys] */
  float* probs = scores + n_keys;           /* [1, n_keys] */
  const long tok_stride = (long)n_head_kv * hd;
  for (int j = 0; j < n_keys; ++j)
    for (int d = 0; d < hd; ++d) kt[(long)d * n_keys + j] = kc[j * tok_stride + (long)kvh * hd + d];
  hl_ref_matmul(q, kt, scores, 1, hd, n_keys);
  const float inv_sqrt = 1.0f / sqrtf((float)hd);
  for (int j = 0; j < n_keys; ++j) scores[j] = scores[j] * inv_sqrt;
  hl_ref_softmax_last_dim(scores, probs, 1, n_keys);
  /* V slice [n_keys, hd] gathered contiguous (slice: glue); reuse kt storage */
  float* vs = kt;
  for (int j = 0; j < n_keys; ++j)
    memcpy(vs + (long)j * hd, vc + j * tok_stride + (long)kvh * hd, sizeof(float) * hd);
  hl_ref_matmul(probs, vs, out, 1, n_keys, hd);
}

/*
 * The whole path for T new tokens of ONE sequence whose cache already holds cur_len tokens:
 * QK-norm (optional) -> RoPE(Q, K) -> append K, V at positions cur_len.. -> causal GQA.
 * Prefill is (cur_len = 0, T = S); a decode step is (T = 1).
 *
 *  q        [T, n_head, hd]      raw query rows (not modified)
 *  k, v     [T, n_head_kv, hd]   raw key / value rows (not modified)
 *  k_cache, v_cache  [max_len, n_head_kv, hd] float32, updated in place; K is stored after
 *           norm and RoPE, V raw (naive.nim:4074-4076).  With kv_fp16 != 0 both are rounded to
 *           fp16 (RN-even) when stored: the "fp16-KV-aware" variant used to tell cache
 *           quantisation error from kernel error.
 *  rows     optional [n_rows][2] = (token index t in [0,T), head h); NULL = every (t, h), in
 *           which case out is [T, n_head, hd]; otherwise out is [n_rows, hd].
 *  q_rot    optional [T, n_head, hd]: receives Q after norm + RoPE.
 * Returns 0, or -1 on a bad argument.
 */
int hl_ref_attn_forward(const float* q, const float* k, const float* v, float* k_cache,
                        float* v_cache, int cur_len, int max_len, int T, int n_head,
                        int n_head_kv, int hd, int rope_dim, const float* theta, int rope_mode,
                        const float* q_norm_w, const float* k_norm_w, float eps, int kv_fp16,
                        const int32_t* rows, long n_rows, float* out, float* q_rot,
                        int n_threads) {
  if (T <= 0 || n_head <= 0 || n_head_kv <= 0 || n_head % n_head_kv != 0) return -1;
  if (cur_len < 0 || cur_len + T > max_len || rope_dim > hd || (rope_dim & 1)) return -1;
  const int group = n_head / n_head_kv;
  const long kv_tok = (long)n_head_kv * hd;
  const long q_tok = (long)n_head * hd;

  /* 1. K: norm -> rope -> (fp16) -> cache; V: (fp16) -> cache */
  for (int t = 0; t < T; ++t) {
    const int pos = cur_len + t;
    for (int h = 0; h < n_head_kv; ++h) {
      float* kd = k_cache + pos * kv_tok + (long)h * hd;
      float* vd = v_cache + pos * kv_tok + (long)h * hd;
      const float* ks = k + t * kv_tok + (long)h * hd;
      const float* vs = v + t * kv_tok + (long)h * hd;
      if (k_norm_w) hl_ref_rmsnorm(ks, k_norm_w, kd, 1, hd, eps);
      else memcpy(kd, ks, sizeof(float) * hd);
      hl_ref_rope_row(kd, rope_dim, theta, pos, rope_mode);
      memcpy(vd, vs, sizeof(float) * hd);
      if (kv_fp16)
        for (int d = 0; d < hd; ++d) {
          kd[d] = hl_ref_round_fp16(kd[d]);
          vd[d] = hl_ref_round_fp16(vd[d]);
        }
    }
  }

  /* 2. attention rows */
  const long total = rows ? n_rows : (long)T * n_head;
  int err = 0;
#ifdef _OPENMP
  if (n_threads > 0) omp_set_num_threads(n_threads);
#pragma omp parallel if (n_threads != 1)
#endif
  {
    const long max_keys = (long)cur_len + T;
    float* scratch = (float*)malloc(sizeof(float) * (2 * max_keys + max_keys * hd + 2L * hd));
    if (!scratch) {
#ifdef _OPENMP
#pragma omp atomic write
#endif
      err = -2;
    } else {
      float* qrow = scratch + 2 * max_keys + max_keys * hd;
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 4)
#endif
      for (long r = 0; r < total; ++r) {
        const int t = rows ? rows[2 * r] : (int)(r / n_head);
        const int h = rows ? rows[2 * r + 1] : (int)(r % n_head);
        const int pos = cur_len + t;
        const float* qs = q + t * q_tok + (long)h * hd;
        if (q_norm_w) hl_ref_rmsnorm(qs, q_norm_w, qrow, 1, hd, eps);
        else memcpy(qrow, qs, sizeof(float) * hd);
        hl_ref_rope_row(qrow, rope_dim, theta, pos, rope_mode);
        if (q_rot) memcpy(q_rot + t * q_tok + (long)h * hd, qrow, sizeof(float) * hd);
        attention_row(qrow, k_cache, v_cache, h / group, n_head_kv, hd, pos + 1,
                      out + r * hd, scratch);
      }
      free(scratch);
    }
  }
  return err;
}

/* Attention output gate of the qwen3.5-MoE layers: dst <- sigmoid(gate) * dst, float32, with
 * sigmoid(g) = 1 / (1 + expf(-g)).  backends/naive.nim:2287-2293 (attnGateKernel), applied to the
 * attention output before the output projection (naive.nim:4259-4260). */
void hl_ref_attn_gate(float* dst, const float* gate, long n) {
  for (long i = 0; i < n; ++i) {
    const float sig = 1.0f / (1.0f + expf(-gate[i]));
    dst[i] = sig * dst[i];
  }
}

int hl_ref_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
