// Split-KV decode attention over the paged fp16 KV cache, plus the log-sum-exp combine.
// Replaces attentionDecodeKernel (src/hippo_leap/backends/naive.nim:3292-3383; warp-per-head prior
// art at backends/megakernel.nim:868-919) together with the Q half of qkNorm / ropeQKDecode.
//
// Work item = (sequence, KV head, context chunk): one CTA streams that chunk's K and V pages ONCE
// and serves all G = n_head / n_head_kv query heads that share the KV head (the reference re-reads
// the cache G times, one block per query head).  HBM-bound: the design goal is bytes in flight.
//   - a producer warp walks the block table and issues one TMA box (16 rows x 64 halfs, 2 KiB,
//     128-byte swizzle) per (page row-group, column half) into a ring of STAGES stages;
//   - NW consumer warps take 16 keys each per stage: S = Q K^T and O += P V on mma.sync.m16n8k16
//     with the G query heads padded to the 16 MMA rows, fp32 online softmax (exp2), quad shuffles
//     for the row max / sum;
//   - the warps' (m, l, O) states are merged through shared memory and written as one partial per
//     chunk (or the final output when the sequence has a single chunk);
//   - attn_combine_kernel merges the chunk partials: out = sum_c 2^(m_c-M) o_c / sum_c 2^(m_c-M) l_c.
#pragma once
#include <cuda.h>

#include "hl_device.cuh"

namespace hl {

struct DecodeArgs {
  View q, out;
  View gate;  // optional sigmoid gate on the output, same indexing as out; ptr == nullptr: none
  const float* q_norm_w;
  const float* theta;
  const int32_t* ctx_lens;
  const int32_t* block_tables;
  float* part_o;   // [batch][n_head][max_chunks][HD]
  float* part_ml;  // [batch][n_head][max_chunks][2]  (m in log2 units, l)
  int32_t* status;
  float eps, scale_log2;  // scale_log2 = log2(e) / sqrt(head_dim)
  int32_t n_head, n_head_kv, group;
  int32_t rope_dim, rope_mode;
  int32_t block_tokens, num_blocks, max_blocks;
  int32_t chunk_tokens, max_chunks;
  // Extra destinations of the output rows (same dtype and strides as `out`): the same buffer on peer GPUs, mapped
  // into this GPU's address space.  With KV heads sharded across GPUs every finished row is stored to all of them
  // with plain stores over NVLink, so the all-gather of head outputs needs no collective kernel.
  void* bcast[7];
  int32_t n_bcast;
  int32_t early_q;  // 1: the query rows are known to be complete before this grid can start (read before the wait)
};

// One output element to the local destination and to every broadcast destination.
__device__ __forceinline__ void decode_store(const DecodeArgs& a, int b, int h, int d, float x) {
  view_store(a.out, b, h, d, x);
  for (int i = 0; i < a.n_bcast; ++i) {
    View o = a.out;
    o.ptr = a.bcast[i];
    view_store(o, b, h, d, x);
  }
}

template <int HD, int NW, int STAGES>
struct DecodeCfg {
  static constexpr int kStageTok = 16 * NW;
  static constexpr int kHalves = HD / 64;
  static constexpr int kHalfBytes = kStageTok * 128;       // one 64-column half of a K or V tile
  static constexpr int kTileBytes = kHalves * kHalfBytes;  // K (or V) of one stage
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kQHalfBytes = 16 * 128;
  static constexpr int kQBytes = kHalves * kQHalfBytes;  // 16 x HD fp16, swizzled
  static constexpr int kMergeBytes = NW * 16 * HD * 4 + NW * 16 * 8;
  static constexpr int kRingBytes = STAGES * kStageBytes;
  static_assert(kRingBytes >= kMergeBytes, "merge buffer reuses the ring");
  static constexpr int kQStageBytes = 16 * HD * 4;  // fp32 staging of the query rows (own area: the ring fills meanwhile)
  static constexpr int kSmemBytes = 1024 /*align slack*/ + kQBytes + kRingBytes + kQStageBytes + 2 * STAGES * 8;
  static constexpr int kThreads = (NW + 1) * 32;
};

template <int HD, int NW, int STAGES>
__global__ void __launch_bounds__((NW + 1) * 32)
    attn_decode_kernel(const __grid_constant__ CUtensorMap k_map,
                       const __grid_constant__ CUtensorMap v_map, DecodeArgs a) {
  using Cfg = DecodeCfg<HD, NW, STAGES>;
  // a kernel queued behind this one with programmatic stream serialisation (an output projection that first
  // prefetches its weights) may start now; it still waits for this whole grid before it reads the attention output
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  // ctx_lens is device data the host cannot see: a value beyond what the grid and the partial slots were sized for
  // (max_ctx_h) is reported and clamped, so the combine pass never reads past this row's slots; a non-positive one
  // (decode always attends at least the new token's own key) is reported and the output row is zeroed.
  // Launched with programmatic stream serialisation this grid starts while the kernel in front (the KV append of the
  // same step) is still running.  What that kernel writes -- the cache -- is only touched after griddepcontrol.wait;
  // the barrier set-up runs before it, and so does the query prologue when the caller vouches for the query rows
  // (early_q: the library's own backends, where the append always sits between the projection and this kernel).  Every thread passes a wait before it exits, so that a
  // grid queued behind this one can rely on everything in front of this one having completed too.
  int ctx = a.ctx_lens[b];
  if (ctx > a.max_chunks * a.chunk_tokens) {
    report(a.status, HL_ERR_BOUNDS, b);
    ctx = a.max_chunks * a.chunk_tokens;
  }
  if (ctx <= 0) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (chunk == 0) {
      report(a.status, HL_ERR_BOUNDS, b);
      for (int idx = threadIdx.x; idx < a.group * HD; idx += blockDim.x)
        decode_store(a, b, kvh * a.group + idx / HD, idx % HD, 0.f);
    }
    return;
  }
  const int t_begin = chunk * a.chunk_tokens;
  if (t_begin >= ctx) {  // uniform for the CTA
    asm volatile("griddepcontrol.wait;" ::: "memory");
    return;
  }
  const int t_end = min(ctx, t_begin + a.chunk_tokens);
  const int n_iter = (t_end - t_begin + Cfg::kStageTok - 1) / Cfg::kStageTok;
  const int n_chunks_seq = (ctx + a.chunk_tokens - 1) / a.chunk_tokens;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_tile = base;
  const uint32_t ring = base + Cfg::kQBytes;
  uint8_t* ring_gen = gen + Cfg::kQBytes;
  float* q_stage = reinterpret_cast<float*>(ring_gen + Cfg::kRingBytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(ring_gen + Cfg::kRingBytes + Cfg::kQStageBytes);
  uint64_t* empty = full + STAGES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NW);
    }
    mbar_fence_init();
  }

  __syncthreads();  // barriers initialised: the producer may start filling the ring at once

  if (warp == NW) {
    // ================= producer warp =================
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the append in front has written this step's K / V rows
    constexpr int kOpsPerGroup = 2 * Cfg::kHalves;  // K halves + V halves of one 16-row group
    constexpr int kOps = NW * kOpsPerGroup;
    static_assert(kOps <= 32, "one lane per TMA box");
    for (int it = 0; it < n_iter; ++it) {
      const int s = it % STAGES;
      if (it >= STAGES) mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, a.status, 100 + s);
      const int tok0 = t_begin + it * Cfg::kStageTok;
      const int n_groups = min(NW, (t_end - tok0 + 15) >> 4);  // 16-row groups holding live keys
      if (lane == 0) mbar_arrive_expect_tx(&full[s], n_groups * kOpsPerGroup * 2048);
      __syncwarp();
      if (lane < kOps) {
        const int grp = lane / kOpsPerGroup, op = lane % kOpsPerGroup;
        if (grp < n_groups) {
          const int tok = tok0 + grp * 16;
          const int lb = tok / a.block_tokens;
          int pb = lb < a.max_blocks
                       ? a.block_tables[static_cast<int64_t>(b) * a.max_blocks + lb]
                       : -1;
          if (pb < 0 || pb >= a.num_blocks) {
            report(a.status, HL_ERR_BOUNDS, b);
            pb = 0;  // stay inside the pool; the status word tells the host
          }
          const int row = (pb * a.n_head_kv + kvh) * a.block_tokens + tok % a.block_tokens;
          const bool is_v = op >= Cfg::kHalves;
          const int hh = is_v ? op - Cfg::kHalves : op;
          const uint32_t dst = ring + s * Cfg::kStageBytes + (is_v ? Cfg::kTileBytes : 0) +
                               hh * Cfg::kHalfBytes + grp * 16 * 128;
          tma_load_2d(dst, is_v ? &v_map : &k_map, &full[s], hh * 64, row);
        }
      }
      __syncwarp();
    }
    return;
  }

  // ================= consumer warps =================
  // ---- Q prologue (while the first K/V stages are in flight): G rows -> norm -> RoPE at pos = ctx-1
  //      -> fp16 swizzled tile (rows >= G zero)
  if (!a.early_q) asm volatile("griddepcontrol.wait;" ::: "memory");  // the query rows may come from the grid in front
  {
    const int pos = ctx - 1;
    for (int r = warp; r < 16; r += NW) {
      float* x = q_stage + r * HD;
      const bool live = r < a.group;
      if (live) {
        const int h = kvh * a.group + r;
#pragma unroll
        for (int d = lane; d < HD; d += 32) x[d] = view_load(a.q, b, h, d);
        __syncwarp();
        norm_rope_row<HD>(x, a.q_norm_w, a.eps, a.theta, a.rope_dim, a.rope_mode, pos, lane);
      }
      store_row_fp16_swz<HD>(q_tile, Cfg::kQHalfBytes, r, x, lane, !live);
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");  // (long since satisfied: the ring cannot fill before it)
  named_bar_sync(2, NW * 32);  // the whole Q tile is written before any warp reads its fragments
  const int g = lane >> 2, tq = lane & 3;
  uint32_t qa[HD / 16][4];
  {
    const int mi = lane >> 3;
    const int row = (mi & 1) * 8 + (lane & 7);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const int chunk16 = (ks & 3) * 2 + (mi >> 1);
      ldsm_x4(swz128(q_tile + (ks >> 2) * Cfg::kQHalfBytes, row, chunk16), qa[ks][0], qa[ks][1],
              qa[ks][2], qa[ks][3]);
    }
  }
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const float c = a.scale_log2;

  for (int it = 0; it < n_iter; ++it) {
    const int s = it % STAGES;
    mbar_wait(&full[s], (it / STAGES) & 1, a.status, 200 + s);
    const int nvalid = t_end - (t_begin + it * Cfg::kStageTok + 16 * warp);
    if (nvalid > 0) {
      const uint32_t k_tile = ring + s * Cfg::kStageBytes;
      const uint32_t v_tile = k_tile + Cfg::kTileBytes;
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const int mi = lane >> 3;
        const int key = 16 * warp + (mi >> 1) * 8 + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          uint32_t b00, b01, b10, b11;
          ldsm_x4(swz128(k_tile + (ks >> 2) * Cfg::kHalfBytes, key, (ks & 3) * 2 + (mi & 1)), b00,
                  b01, b10, b11);
          mma16816(sc[0], qa[ks], b00, b01);
          mma16816(sc[1], qa[ks], b10, b11);
        }
      }
      if (nvalid < 16) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (nt * 8 + 2 * tq + (e & 1) >= nvalid) sc[nt][e] = -INFINITY;
      }
      float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
      float mx1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float corr0 = fast_exp2((m0 - mn0) * c), corr1 = fast_exp2((m1 - mn1) * c);
      m0 = mn0;
      m1 = mn1;
      const float ms0 = mn0 * c, ms1 = mn1 * c;
      float p[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        p[nt][0] = fast_exp2(fmaf(sc[nt][0], c, -ms0));
        p[nt][1] = fast_exp2(fmaf(sc[nt][1], c, -ms0));
        p[nt][2] = fast_exp2(fmaf(sc[nt][2], c, -ms1));
        p[nt][3] = fast_exp2(fmaf(sc[nt][3], c, -ms1));
      }
      l0 = l0 * corr0 + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
      l1 = l1 * corr1 + (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
      uint32_t pa[4];
      pa[0] = pack_half2(p[0][0], p[0][1]);
      pa[1] = pack_half2(p[0][2], p[0][3]);
      pa[2] = pack_half2(p[1][0], p[1][1]);
      pa[3] = pack_half2(p[1][2], p[1][3]);
      {
        const int mi = lane >> 3;
        const int key = 16 * warp + (mi & 1) * 8 + (lane & 7);
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {  // pairs of 8-wide d tiles
          uint32_t b00, b01, b10, b11;
          ldsm_x4_t(swz128(v_tile + (dp >> 2) * Cfg::kHalfBytes, key, (dp & 3) * 2 + (mi >> 1)),
                    b00, b01, b10, b11);
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            o[2 * dp + e][0] *= corr0;
            o[2 * dp + e][1] *= corr0;
            o[2 * dp + e][2] *= corr1;
            o[2 * dp + e][3] *= corr1;
          }
          mma16816(o[2 * dp], pa, b00, b01);
          mma16816(o[2 * dp + 1], pa, b10, b11);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // ---- merge the NW warp states through the (now idle) ring ---------------------------------
  named_bar_sync(1, NW * 32);
  float* mo = reinterpret_cast<float*>(ring_gen);        // [NW][16][HD]
  float* mml = mo + NW * 16 * HD;                         // [NW][16][2]
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) {
    const int d = nt * 8 + 2 * tq;
    *reinterpret_cast<float2*>(mo + (warp * 16 + g) * HD + d) = make_float2(o[nt][0], o[nt][1]);
    *reinterpret_cast<float2*>(mo + (warp * 16 + g + 8) * HD + d) = make_float2(o[nt][2], o[nt][3]);
  }
  if (tq == 0) {
    mml[(warp * 16 + g) * 2 + 0] = m0 * c;
    mml[(warp * 16 + g) * 2 + 1] = l0;
    mml[(warp * 16 + g + 8) * 2 + 0] = m1 * c;
    mml[(warp * 16 + g + 8) * 2 + 1] = l1;
  }
  named_bar_sync(1, NW * 32);
  for (int idx = tid; idx < a.group * HD; idx += NW * 32) {
    const int r = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, mml[(w * 16 + r) * 2]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float f = fast_exp2(mml[(w * 16 + r) * 2] - M);
      L += mml[(w * 16 + r) * 2 + 1] * f;
      acc += mo[(w * 16 + r) * HD + d] * f;
    }
    const int h = kvh * a.group + r;
    if (n_chunks_seq == 1) {
      decode_store(a, b, h, d, apply_gate(a.gate, b, h, d, acc / L));
    } else {
      const int64_t pi = (static_cast<int64_t>(b) * a.n_head + h) * a.max_chunks + chunk;
      a.part_o[pi * HD + d] = acc;
      if (d == 0) {
        a.part_ml[pi * 2] = M;
        a.part_ml[pi * 2 + 1] = L;
      }
    }
  }
}

// Second pass of split-KV: merge the chunk partials of one (sequence, head).
template <int HD>
__global__ void __launch_bounds__(HD) attn_combine_kernel(DecodeArgs a) {
  // a kernel queued behind this one with programmatic stream serialisation (the output projection's GEMV) may start
  // its weight prefetch now; it still waits for this grid to finish before it reads the attention output
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the decode grid in front has written the partials
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int ctx = min(a.ctx_lens[b], a.max_chunks * a.chunk_tokens);  // clamped (and reported) like the decode kernel
  const int n = (ctx + a.chunk_tokens - 1) / a.chunk_tokens;
  if (n <= 1) return;  // the decode kernel already wrote the final row (or zeroed it: empty context)
  const int64_t p0 = (static_cast<int64_t>(b) * a.n_head + h) * a.max_chunks;
  // Eight partials per trip: their (max, sum) pairs and this thread's output element are all requested before any is
  // used, so a trip costs one L2 round trip.  (One partial per trip, each load waited for before the next was issued,
  // made this pass a chain of n round trips: longer than the decode kernel itself for a single 2k-token sequence.)
  float M = -INFINITY, L = 0.f, acc = 0.f;
  for (int base = 0; base < n; base += 8) {
    float m8[8], l8[8], o8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool ok = base + i < n;
      const int64_t pi = p0 + base + i;
      m8[i] = -INFINITY;  // a missing partial weighs exp2(-inf) = 0
      l8[i] = o8[i] = 0.f;
      if (ok) {           // (predicated loads: nothing is fetched for a missing partial)
        const float2 ml = *reinterpret_cast<const float2*>(a.part_ml + pi * 2);
        m8[i] = ml.x;
        l8[i] = ml.y;
        o8[i] = a.part_o[pi * HD + d];
      }
    }
    float Mt = M;
#pragma unroll
    for (int i = 0; i < 8; ++i) Mt = fmaxf(Mt, m8[i]);
    if (base > 0) {  // bring what was summed so far to the new maximum
      const float f = exp2f(M - Mt);
      L *= f;
      acc *= f;
    }
    M = Mt;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = exp2f(m8[i] - M);
      L += l8[i] * f;
      acc += o8[i] * f;
    }
  }
  decode_store(a, b, h, d, apply_gate(a.gate, b, h, d, acc / L));
}

}  // namespace hl
