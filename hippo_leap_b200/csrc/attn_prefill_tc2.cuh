// Causal GQA prefill, head_dim 128, on PAIRS of SMs: tcgen05.mma.cta_group::2.
//
// The single-SM kernel (attn_prefill_tc.cuh) re-reads every K/V block from L2 once per 256 query
// rows; at 32k tokens that L2 -> shared-memory stream, not the tensor core, bounds it.  Here two
// CTAs of a cluster work as one: each holds 2 x 128 query rows (two ping-pong tiles, as before) and
// loads only HALF of every K/V block -- CTA r the keys [64r, 64r+64) of the K block and the value
// columns [64r, 64r+64) of the V block -- and one thread of the leader CTA issues MMAs of M = 256
// that read the A operand (Q rows, or P in TMEM) from both CTAs and the two halves of B from both
// shared memories.  A K/V block is therefore fetched once per 512 query rows, and each SM's shared
// memory sees half the operand traffic.
//
//   per CTA: warps 0-3 / 4-7 softmax of tile A / B (one thread per row), warp 8 TMA producer,
//            warp 9 TMEM owner (+ MMA issuer in the leader), warps 10-11 idle
//   leader-only barriers : q_ready (512 arrivals: both CTAs' softmax threads), p_full[t] (256),
//                          k_full / v_full (the leader posts the expected bytes of BOTH halves; the
//                          peer's TMA completes on the leader's barrier through the cta_group::2 form)
//   both-CTA barriers    : s_full[t], o_full[t], k_empty[s], v_empty[s], signalled in both CTAs at
//                          once by tcgen05.commit with a CTA mask
// No TMA multicast is used anywhere.  Every wait is bounded; TMEM is released on every path.
#pragma once
#include <cuda.h>

#include "attn_prefill_tc.cuh"

namespace hl {

struct PrefillTc2Cfg {
  static constexpr int HD = 128;
  static constexpr int kStages = 4;
  static constexpr int kQHalfBytes = 128 * 128;       // 128 query rows x 64 halfs
  static constexpr int kQTileBytes = 2 * kQHalfBytes;  // 32 KiB per tile
  static constexpr int kKHalfBytes = 64 * 128;        // this CTA's 64 keys x 64 halfs
  static constexpr int kKStageBytes = 2 * kKHalfBytes;  // 16 KiB: 64 keys x 128 dims
  static constexpr int kVStageBytes = 128 * 128;      // 16 KiB: 128 keys x this CTA's 64 value columns
  static constexpr int kQOff = 0;
  static constexpr int kKOff = 2 * kQTileBytes;
  static constexpr int kVOff = kKOff + kStages * kKStageBytes;
  static constexpr int kRowOff = kVOff + kStages * kVStageBytes;
  static constexpr int kBarOff = kRowOff + 8 * HD * 4;
  static constexpr int kNumBars = 4 * kStages + 7;
  static constexpr int kSmemBytes = 1024 + kBarOff + kNumBars * 8 + 16;
  static constexpr int kThreads = 384;
  static constexpr int kTmemCols = 512;
  static constexpr uint32_t kColS = 0, kColO = 256;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(smem_u32(bar)),
      "r"(rank)
      : "memory");
}
// tcgen05.commit that arrives on the barrier at this offset in BOTH CTAs of the pair
__device__ __forceinline__ void tc2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}
__device__ __forceinline__ void tc2_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc2_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// TMA load into THIS CTA's shared memory whose completion bytes are counted on the LEADER CTA's
// barrier (same offset, CTA-pair bit cleared).  No multicast.
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const void* tmap, uint64_t* bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar) & 0xFEFFFFFFu), "r"(c0), "r"(c1)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(384, 1)
    attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                            PrefillTcArgs ta) {
  using Cfg = PrefillTc2Cfg;
  constexpr int HD = 128;
  constexpr int S = Cfg::kStages;
  const PrefillArgs& a = ta.p;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = (gridDim.x >> 1) - 1 - (blockIdx.x >> 1);  // longest first
  const int h = blockIdx.y;
  const int kvh = h / a.group;
  const int t0 = pair * 512;  // first query row of the pair; tile t covers rows [t0 + 256 t, +256)

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + Cfg::kBarOff);
  uint64_t* k_full = bars;
  uint64_t* k_empty = bars + S;
  uint64_t* v_full = bars + 2 * S;
  uint64_t* v_empty = bars + 3 * S;
  uint64_t* s_full = bars + 4 * S;
  uint64_t* p_full = bars + 4 * S + 2;
  uint64_t* o_full = bars + 4 * S + 4;
  uint64_t* q_ready = bars + 4 * S + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // keys attended by tile t of the PAIR: [0, k_end[t]); both CTAs run the same number of blocks
  int k_end[2], n_blk[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int live = min(256, a.n_tok - (t0 + 256 * t));
    k_end[t] = live > 0 ? a.start_pos + t0 + 256 * t + live : 0;
    n_blk[t] = (k_end[t] + 127) >> 7;
  }
  const int n_max = max(n_blk[0], n_blk[1]);
  const int k_end_max = max(k_end[0], k_end[1]);

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 256);  // 128 rows of this tile in each CTA
      mbar_init(&o_full[t], 1);
    }
    mbar_init(q_ready, 512);
    *abort_flag = (a.status != nullptr && *a.status != 0) ? 1 : 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(Cfg::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anything can arrive on them
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8) {
    // ======================= TMA producer (both CTAs) =======================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    for (int j = 0; j < n_max; ++j) {
      const int s = j % S;
      const uint32_t par = ((j / S) - 1) & 1;
      // K half of this CTA: keys [128 j + 64 rank, +64): 4 groups of 16 rows x 2 column halves (lanes 0-7)
      // V half of this CTA: keys [128 j, +128), columns [64 rank, +64): 8 groups of 16 rows (lanes 8-15)
      int row = static_cast<int>(ta.oob_row);
      int tok = -1;
      if (lane < 8) tok = j * 128 + 64 * static_cast<int>(rank) + (lane >> 1) * 16;
      else if (lane < 16) tok = j * 128 + (lane - 8) * 16;
      if (tok >= 0 && tok < k_end_max) {
        const int lb = tok / a.block_tokens;
        int pb = lb < a.n_blocks_in_table ? a.block_table[lb] : -1;
        if (pb < 0 || pb >= a.num_blocks) {
          report(a.status, HL_ERR_BOUNDS, lb);
          pb = 0;
        }
        row = (pb * a.n_head_kv + kvh) * a.block_tokens + tok % a.block_tokens;
      }
      if (j >= S) tc_wait(&k_empty[s], par, a.status, 600 + s, abort_flag);
      if (leader && lane == 0) mbar_arrive_expect_tx(&k_full[s], 2 * Cfg::kKStageBytes);
      __syncwarp();
      if (lane < 8)
        tma2_load_2d(base + Cfg::kKOff + s * Cfg::kKStageBytes + (lane & 1) * Cfg::kKHalfBytes + (lane >> 1) * 2048,
                     &k_map, &k_full[s], (lane & 1) * 64, row);
      if (j >= S) tc_wait(&v_empty[s], par, a.status, 610 + s, abort_flag);
      if (leader && lane == 0) mbar_arrive_expect_tx(&v_full[s], 2 * Cfg::kVStageBytes);
      __syncwarp();
      if (lane >= 8 && lane < 16)
        tma2_load_2d(base + Cfg::kVOff + s * Cfg::kVStageBytes + (lane - 8) * 2048, &v_map, &v_full[s],
                     64 * static_cast<int>(rank), row);
      __syncwarp();
    }
  } else if (warp == 9) {
    // ======================= MMA issuer (leader CTA only) =======================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (leader && lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(256, 128, 0);
      constexpr uint32_t idesc_pv = umma_idesc(256, HD, 1);
      auto issue_qk = [&](int t, int j) {
        const uint32_t a_base = base + Cfg::kQOff + t * Cfg::kQTileBytes;
        const uint32_t b_base = base + Cfg::kKOff + (j % S) * Cfg::kKStageBytes;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          tc2_mma_ss(tmem + Cfg::kColS + t * 128,
                     umma_desc(a_base + (ks >> 2) * Cfg::kQHalfBytes + (ks & 3) * 32, 16, 1024),
                     umma_desc(b_base + (ks >> 2) * Cfg::kKHalfBytes + (ks & 3) * 32, 16, 1024), idesc_qk,
                     ks > 0 ? 1u : 0u);
      };
      auto issue_pv = [&](int t, int j) {
        const uint32_t b_base = base + Cfg::kVOff + (j % S) * Cfg::kVStageBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          tc2_mma_ts(tmem + Cfg::kColO + t * HD, tmem + Cfg::kColS + t * 128 + ks * 8,
                     umma_desc(b_base + ks * 2048, Cfg::kVStageBytes, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
      };
      tc_wait(q_ready, 0, a.status, 620, abort_flag);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_after();
      if (n_max > 0) {
        tc_wait(&k_full[0], 0, a.status, 621, abort_flag);
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (n_blk[t] > 0) {
            issue_qk(t, 0);
            tc2_commit_both(&s_full[t]);
          }
        tc2_commit_both(&k_empty[0]);
      }
      for (int j = 0; j < n_max; ++j) {
        bool next_qk = false;
        for (int t = 0; t < 2; ++t) {
          if (j >= n_blk[t]) continue;
          tc_wait(&p_full[t], j & 1, a.status, 630 + t, abort_flag);
          tc_wait(&v_full[j % S], (j / S) & 1, a.status, 632, abort_flag);
          tc_fence_after();
          issue_pv(t, j);
          if (j + 1 < n_blk[t]) {
            tc_wait(&k_full[(j + 1) % S], ((j + 1) / S) & 1, a.status, 633, abort_flag);
            tc_fence_after();
            issue_qk(t, j + 1);
            tc2_commit_both(&s_full[t]);
            next_qk = true;
          } else {
            tc2_commit_both(&o_full[t]);
          }
        }
        tc2_commit_both(&v_empty[j % S]);
        if (next_qk) tc2_commit_both(&k_empty[(j + 1) % S]);
      }
    }
    __syncwarp();
  } else if (warp >= 10) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  } else {
    // ======================= softmax warps: tile t, row r of THIS CTA =======================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int t = warp >> 2;
    const int r = tid & 127;
    const int row0 = t0 + 256 * t + 128 * static_cast<int>(rank);  // first token of this CTA's rows of tile t
    const int trow = row0 + r;
    const int pos = a.start_pos + trow;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_sel + Cfg::kColS + t * 128;
    const uint32_t tO = tmem + lane_sel + Cfg::kColO + t * HD;

    // ---- Q prologue: this warp prepares rows [32*(warp&3), +32) of tile t ----
    {
      const uint32_t q_tile = base + Cfg::kQOff + t * Cfg::kQTileBytes;
      constexpr int VEC = HD / 32;
      const bool fast = a.q.ds == 1 && a.rope_dim == HD && ta.cs_table != nullptr;
      float* xrow = reinterpret_cast<float*>(gen + Cfg::kRowOff) + warp * HD;
      if (fast) {
        constexpr int R = 8;
        const int d0 = lane * VEC;
        const int last_pos = a.start_pos + a.n_tok - 1;
        for (int rb = 0; rb < 32; rb += R) {
          float x[R][VEC];
          float2 cs[R][VEC];
#pragma unroll
          for (int u = 0; u < R; ++u) {
            const int tt = row0 + (warp & 3) * 32 + rb + u;
            if (tt < a.n_tok) {
              load_vec<VEC>(a.q, tt, h, d0, x[u]);
            } else {
#pragma unroll
              for (int e = 0; e < VEC; ++e) x[u][e] = 0.f;
            }
            const float2* csr = ta.cs_table + static_cast<int64_t>(min(a.start_pos + tt, last_pos)) * (HD / 2);
            if (a.rope_mode == HL_ROPE_INTERLEAVED) {
#pragma unroll
              for (int e = 0; e < VEC; e += 2) cs[u][e >> 1] = csr[(d0 + e) >> 1];
            } else {
#pragma unroll
              for (int e = 0; e < VEC; ++e) cs[u][e] = csr[(d0 + e) & (HD / 2 - 1)];
            }
          }
          if (a.q_norm_w != nullptr) {
            float w[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) w[e] = a.q_norm_w[d0 + e];
#pragma unroll
            for (int u = 0; u < R; ++u) {
              float ss = 0.f;
#pragma unroll
              for (int e = 0; e < VEC; ++e) ss += x[u][e] * x[u][e];
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
              const float inv = 1.0f / sqrtf(ss / static_cast<float>(HD) + a.eps);
#pragma unroll
              for (int e = 0; e < VEC; ++e) x[u][e] = x[u][e] * inv * w[e];
            }
          }
#pragma unroll
          for (int u = 0; u < R; ++u) {
            if (a.rope_mode == HL_ROPE_INTERLEAVED) {
#pragma unroll
              for (int e = 0; e < VEC; e += 2) {
                const float2 c = cs[u][e >> 1];
                const float v0 = x[u][e], v1 = x[u][e + 1];
                x[u][e] = v0 * c.x - v1 * c.y;
                x[u][e + 1] = v0 * c.y + v1 * c.x;
              }
            } else {
#pragma unroll
              for (int e = 0; e < VEC; ++e) {
                const float other = __shfl_xor_sync(0xffffffffu, x[u][e], 16);
                const float2 c = cs[u][e];
                x[u][e] = (d0 + e < HD / 2) ? x[u][e] * c.x - other * c.y : other * c.y + x[u][e] * c.x;
              }
            }
            const int row = (warp & 3) * 32 + rb + u;
            const uint32_t addr = swz128(q_tile + (d0 >> 6) * Cfg::kQHalfBytes, row, (d0 & 63) >> 3) + (d0 & 7) * 2;
            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(pack_half2(x[u][0], x[u][1])),
                         "r"(pack_half2(x[u][2], x[u][3]))
                         : "memory");
          }
        }
      } else {
        for (int rr = 0; rr < 32; ++rr) {
          const int row = (warp & 3) * 32 + rr;
          const int tt = row0 + row;
          const bool live = tt < a.n_tok;
          if (live) {
#pragma unroll
            for (int d = lane; d < HD; d += 32) xrow[d] = view_load(a.q, tt, h, d);
            __syncwarp();
            norm_rope_row<HD>(xrow, a.q_norm_w, a.eps, a.theta, a.rope_dim, a.rope_mode, a.start_pos + tt, lane);
          }
          store_row_fp16_swz<HD>(q_tile, Cfg::kQHalfBytes, row, xrow, lane, !live);
          __syncwarp();
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive_cluster(q_ready, 0);
    }

    float m = -INFINITY, l = 0.f;
    const float c = a.scale_log2;
    for (int j = 0; j < n_blk[t]; ++j) {
      float s[128];
      tc_wait(&s_full[t], j & 1, a.status, 640 + t, abort_flag);
      tc_fence_after();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) tc_ld32f(tS + q4 * 32, s + q4 * 32);
      tc_wait_ld();
      const int key0 = j * 128;
      if (key0 + 127 > a.start_pos + row0) {  // block touches the diagonal of this CTA's rows
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (key0 + i > pos) s[i] = -INFINITY;
      }
      float mx;
      {
        float m4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
        for (int i = 4; i < 128; i += 8) {
          m4[0] = max3(m4[0], s[i], s[i + 1]);
          m4[1] = max3(m4[1], s[i + 2], s[i + 3]);
          if (i + 4 < 128) {
            m4[2] = max3(m4[2], s[i + 4], s[i + 5]);
            m4[3] = max3(m4[3], s[i + 6], s[i + 7]);
          }
        }
        mx = fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]);
      }
      if (j == 0) {
        m = mx;  // block 0 always holds key 0 <= pos, so the maximum is finite from here on
      } else {
        // A block wholly above this row's diagonal (the upper CTA's last block) gives mx = -inf: no rescale.
        const bool need = (mx - m) * c > 8.0f;
        if (__any_sync(0xffffffffu, need)) {
          const float f = need ? fast_exp2((m - mx) * c) : 1.0f;
          if (need) m = mx;
          l *= f;
#pragma unroll
          for (int q4 = 0; q4 < HD / 32; ++q4) {
            float oreg[32];
            tc_ld32f(tO + q4 * 32, oreg);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) oreg[i] *= f;
            tc_st32f(tO + q4 * 32, oreg);
          }
          tc_wait_st();
        }
      }
      const float mc = m * c;
      const uint64_t c2 = pack_f32x2(c, c), nmc2 = pack_f32x2(-mc, -mc);
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
      uint32_t pk[64];
#pragma unroll
      for (int half_i = 0; half_i < 2; ++half_i) {
#pragma unroll
        for (int i = half_i * 64; i < half_i * 64 + 64; i += 2) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(s[i], s[i + 1]), c2, nmc2), x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          sum2[(i >> 1) & 3] = add_f32x2(sum2[(i >> 1) & 3], pack_f32x2(p0, p1));
          pk[i >> 1] = pack_half2(p0, p1);
        }
        tc_st32(tS + half_i * 32, pk + half_i * 32);
      }
      {
        float a0, a1;
        unpack_f32x2(add_f32x2(add_f32x2(sum2[0], sum2[1]), add_f32x2(sum2[2], sum2[3])), a0, a1);
        l += a0 + a1;
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive_cluster(&p_full[t], 0);
    }
    // ---- epilogue: O / l -> out ----
    if (n_blk[t] > 0) {
      tc_wait(&o_full[t], 0, a.status, 650 + t, abort_flag);
      tc_fence_after();
      const float inv = 1.0f / l;
      const bool live = trow < a.n_tok;
#pragma unroll
      for (int q4 = 0; q4 < HD / 32; ++q4) {
        float oreg[32];
        tc_ld32f(tO + q4 * 32, oreg);
        tc_wait_ld();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; ++i) oreg[i] *= inv;
          if (a.gate.ptr != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i) oreg[i] = apply_gate(a.gate, trow, h, q4 * 32 + i, oreg[i]);
          }
          const int64_t off = static_cast<int64_t>(trow) * a.out.ts + static_cast<int64_t>(h) * a.out.hs + q4 * 32;
          for (int dsti = 0; dsti <= ta.n_bcast; ++dsti) {
            void* obase = dsti == 0 ? const_cast<void*>(a.out.ptr) : ta.bcast[dsti - 1];
            if (a.out.ds == 1 && a.out.dtype == HL_DTYPE_F16 &&
                (reinterpret_cast<uintptr_t>(static_cast<__half*>(obase) + off) & 15) == 0) {
              __half* dst = static_cast<__half*>(obase) + off;
#pragma unroll
              for (int i = 0; i < 32; i += 8)
                *reinterpret_cast<uint4*>(dst + i) =
                    make_uint4(pack_half2(oreg[i], oreg[i + 1]), pack_half2(oreg[i + 2], oreg[i + 3]),
                               pack_half2(oreg[i + 4], oreg[i + 5]), pack_half2(oreg[i + 6], oreg[i + 7]));
            } else if (a.out.ds == 1 && a.out.dtype == HL_DTYPE_F32 &&
                       (reinterpret_cast<uintptr_t>(static_cast<float*>(obase) + off) & 15) == 0) {
              float* dst = static_cast<float*>(obase) + off;
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<float4*>(dst + i) = make_float4(oreg[i], oreg[i + 1], oreg[i + 2], oreg[i + 3]);
            } else {
              View ov = a.out;
              ov.ptr = obase;
#pragma unroll
              for (int i = 0; i < 32; ++i) view_store(ov, trow, h, q4 * 32 + i, oreg[i]);
            }
          }
        }
      }
    }
  }

  // ---- teardown: both CTAs are done with each other's shared memory and TMEM; release TMEM ----
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::kTmemCols) : "memory");
  }
}

}  // namespace hl

// The pair kernel takes head_dim 128 and any n_tok; it pays off once a launch has enough 512-row pairs.
inline bool hl_prefill_tc2_supported(const hl::PrefillArgs& a, int head_dim) { return head_dim == 128 && a.n_tok >= 1; }

static int32_t hl_launch_prefill_tc2(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl::PrefillArgs& a,
                                     void* const* bcast, int n_bcast) {
  using namespace hl;
  using Cfg = PrefillTc2Cfg;
  auto kern = attn_prefill_tc2_kernel;
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    HL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured[ctx->device & 15] = true;
  }
  PrefillTcArgs ta{};
  int32_t rc = hl_prefill_tc_fill_args(ctx, kv, a, 128, bcast, n_bcast, &ta);
  if (rc != HL_OK) return rc;
  ta.box_rows = 16;
  dim3 grid(2 * ((a.n_tok + 511) / 512), a.n_head);
  kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, ctx->stream>>>(kv->k_map[layer], kv->v_map[layer], ta);
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  return HL_OK;
}
