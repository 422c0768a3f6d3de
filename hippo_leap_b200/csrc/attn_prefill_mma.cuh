// Causal GQA prefill on warp-level MMA (mma.sync.m16n8k16): flash-style tiling with an fp32 online
// softmax.  Replaces qkNormPrefill(Q) + ropeAtPos(Q) + attentionPrefillKernel of the reference
// (src/hippo_leap/backends/naive.nim:2928-2971, 3006-3044, 3385-3464), without its 4096-key shared
// memory row (naive.nim:3404) and with start_pos != 0 allowed.
//
// This is the general-shape kernel (any n_tok, start_pos, block size, head_dim 64/128) and the
// on-device cross-check for the tcgen05 kernel, which takes over the large aligned shapes.
//   CTA  = (128-row query tile, query head); 8 consumer warps x 16 rows + 1 TMA producer warp.
//   Q    : raw rows -> (RMSNorm) -> RoPE -> fp16, once per CTA, kept in registers as A fragments.
//   K, V : 64-key stages from the paged cache by TMA (16-row boxes, 128-byte swizzle).
//   Tiles above the diagonal are skipped; the diagonal tiles are masked by index.
//   Large query tiles are scheduled first (longest-first) to balance the causal triangle.
#pragma once
#include <cuda.h>

#include "hl_device.cuh"

namespace hl {

struct PrefillArgs {
  View q, out;
  View gate;  // optional sigmoid gate on the output, same indexing as out; ptr == nullptr: none
  const float* q_norm_w;
  const float* theta;
  const int32_t* block_table;
  int32_t* status;
  float eps, scale_log2;
  int32_t n_tok, start_pos;
  int32_t n_head, n_head_kv, group;
  int32_t rope_dim, rope_mode;
  int32_t block_tokens, num_blocks, n_blocks_in_table;
};

template <int HD, int NW, int STAGES>
struct PrefillMmaCfg {
  static constexpr int kBM = 16 * NW;
  static constexpr int kBN = 64;
  static constexpr int kHalves = HD / 64;
  static constexpr int kHalfBytes = kBN * 128;
  static constexpr int kTileBytes = kHalves * kHalfBytes;
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kQHalfBytes = kBM * 128;
  static constexpr int kQBytes = kHalves * kQHalfBytes;
  static constexpr int kRingBytes = STAGES * kStageBytes;
  static constexpr int kStageF32 = (NW + 1) * HD * 4;  // one fp32 row per warp for the prologue
  static constexpr int kSmemBytes = 1024 + kQBytes + kRingBytes + kStageF32 + 2 * STAGES * 8;
};

template <int HD, int NW, int STAGES>
__global__ void __launch_bounds__((NW + 1) * 32)
    attn_prefill_mma_kernel(const __grid_constant__ CUtensorMap k_map,
                            const __grid_constant__ CUtensorMap v_map, PrefillArgs a) {
  using Cfg = PrefillMmaCfg<HD, NW, STAGES>;
  const int q_tile_idx = gridDim.y - 1 - blockIdx.y;  // heads fastest, query tiles longest first over the whole grid
  const int h = blockIdx.x;
  const int kvh = h / a.group;
  const int t0 = q_tile_idx * Cfg::kBM;
  const int rows_live = min(Cfg::kBM, a.n_tok - t0);
  const int k_end = a.start_pos + t0 + rows_live;  // keys [0, k_end) are attended by this tile
  const int n_iter = (k_end + Cfg::kBN - 1) / Cfg::kBN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_tile = base;
  const uint32_t ring = base + Cfg::kQBytes;
  float* rowbuf = reinterpret_cast<float*>(gen + Cfg::kQBytes + Cfg::kRingBytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(gen + Cfg::kQBytes + Cfg::kRingBytes + Cfg::kStageF32);
  uint64_t* empty = full + STAGES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NW);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == NW) {
    // ================= producer warp =================
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    constexpr int kOpsPerGroup = 2 * Cfg::kHalves;
    constexpr int kOps = 4 * kOpsPerGroup;  // four 16-row groups per 64-key stage
    for (int it = 0; it < n_iter; ++it) {
      const int s = it % STAGES;
      if (it >= STAGES) mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, a.status, 300 + s);
      const int tok0 = it * Cfg::kBN;
      const int n_groups = min(4, (k_end - tok0 + 15) >> 4);
      if (lane == 0) mbar_arrive_expect_tx(&full[s], n_groups * kOpsPerGroup * 2048);
      __syncwarp();
      if (lane < kOps) {
        const int grp = lane / kOpsPerGroup, op = lane % kOpsPerGroup;
        if (grp < n_groups) {
          const int tok = tok0 + grp * 16;
          const int lb = tok / a.block_tokens;
          int pb = lb < a.n_blocks_in_table ? a.block_table[lb] : -1;
          if (pb < 0 || pb >= a.num_blocks) {
            report(a.status, HL_ERR_BOUNDS, lb);
            pb = 0;
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
  // Q prologue for this warp's own 16 rows (no CTA-wide sync needed: each warp only ever reads the
  // rows it wrote).
  {
    float* x = rowbuf + warp * HD;
    for (int r = 0; r < 16; ++r) {
      const int row = warp * 16 + r;
      const int t = t0 + row;
      const bool live = t < a.n_tok;
      if (live) {
#pragma unroll
        for (int d = lane; d < HD; d += 32) x[d] = view_load(a.q, t, h, d);
        __syncwarp();
        norm_rope_row<HD>(x, a.q_norm_w, a.eps, a.theta, a.rope_dim, a.rope_mode, a.start_pos + t,
                          lane);
      }
      store_row_fp16_swz<HD>(q_tile, Cfg::kQHalfBytes, row, x, lane, !live);
      __syncwarp();
    }
  }
  const int g = lane >> 2, tq = lane & 3;
  uint32_t qa[HD / 16][4];
  {
    const int mi = lane >> 3;
    const int row = warp * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
      ldsm_x4(swz128(q_tile + (ks >> 2) * Cfg::kQHalfBytes, row, (ks & 3) * 2 + (mi >> 1)),
              qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
  }
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const float c = a.scale_log2;
  // positions of this thread's two rows, and the last key any row of the warp may see
  const int pos0 = a.start_pos + t0 + warp * 16 + g;
  const int pos1 = pos0 + 8;
  const int warp_last_key = min(a.start_pos + t0 + warp * 16 + 15, k_end - 1);

  for (int it = 0; it < n_iter; ++it) {
    const int s = it % STAGES;
    mbar_wait(&full[s], (it / STAGES) & 1, a.status, 400 + s);
    const int key0 = it * Cfg::kBN;
    if (key0 <= warp_last_key) {
      const uint32_t k_tile = ring + s * Cfg::kStageBytes;
      const uint32_t v_tile = k_tile + Cfg::kTileBytes;
      float sc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
      {
        const int mi = lane >> 3;
        const int krow = (mi >> 1) * 8 + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
          for (int np = 0; np < 4; ++np) {
            uint32_t b00, b01, b10, b11;
            ldsm_x4(swz128(k_tile + (ks >> 2) * Cfg::kHalfBytes, np * 16 + krow,
                           (ks & 3) * 2 + (mi & 1)),
                    b00, b01, b10, b11);
            mma16816(sc[2 * np], qa[ks], b00, b01);
            mma16816(sc[2 * np + 1], qa[ks], b10, b11);
          }
        }
      }
      if (key0 + Cfg::kBN - 1 > a.start_pos + t0 + warp * 16) {  // tile touches the diagonal
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key0 + nt * 8 + 2 * tq + (e & 1);
            if (key > ((e & 2) ? pos1 : pos0)) sc[nt][e] = -INFINITY;
          }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      // Row 0 of a sequence always sees key 0 in the first tile, so the running max is finite
      // from the first tile on and (m - m_new) never evaluates inf - inf.
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float corr0 = fast_exp2((m0 - mn0) * c), corr1 = fast_exp2((m1 - mn1) * c);
      m0 = mn0;
      m1 = mn1;
      const float ms0 = mn0 * c, ms1 = mn1 * c;
      float rs0 = 0.f, rs1 = 0.f;
      uint32_t pa[4][4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        float p[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int nt = 2 * kk + j;
          p[j][0] = fast_exp2(fmaf(sc[nt][0], c, -ms0));
          p[j][1] = fast_exp2(fmaf(sc[nt][1], c, -ms0));
          p[j][2] = fast_exp2(fmaf(sc[nt][2], c, -ms1));
          p[j][3] = fast_exp2(fmaf(sc[nt][3], c, -ms1));
          rs0 += p[j][0] + p[j][1];
          rs1 += p[j][2] + p[j][3];
        }
        pa[kk][0] = pack_half2(p[0][0], p[0][1]);
        pa[kk][1] = pack_half2(p[0][2], p[0][3]);
        pa[kk][2] = pack_half2(p[1][0], p[1][1]);
        pa[kk][3] = pack_half2(p[1][2], p[1][3]);
      }
      l0 = l0 * corr0 + rs0;
      l1 = l1 * corr1 + rs1;
#pragma unroll
      for (int nt = 0; nt < HD / 8; ++nt) {
        o[nt][0] *= corr0;
        o[nt][1] *= corr0;
        o[nt][2] *= corr1;
        o[nt][3] *= corr1;
      }
      {
        const int mi = lane >> 3;
        const int krow = (mi & 1) * 8 + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          // 16-key groups that start at or after k_end were never loaded: P is zero there, and
          // skipping them keeps stale shared memory out of the accumulators.
          if (key0 + kk * 16 < k_end) {
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
              uint32_t b00, b01, b10, b11;
              ldsm_x4_t(swz128(v_tile + (dp >> 2) * Cfg::kHalfBytes, kk * 16 + krow,
                               (dp & 3) * 2 + (mi >> 1)),
                        b00, b01, b10, b11);
              mma16816(o[2 * dp], pa[kk], b00, b01);
              mma16816(o[2 * dp + 1], pa[kk], b10, b11);
            }
          }
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
  const int tr0 = t0 + warp * 16 + g, tr1 = tr0 + 8;
  const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) {
    const int d = nt * 8 + 2 * tq;
    if (tr0 < a.n_tok) {
      view_store(a.out, tr0, h, d, apply_gate(a.gate, tr0, h, d, o[nt][0] * inv0));
      view_store(a.out, tr0, h, d + 1, apply_gate(a.gate, tr0, h, d + 1, o[nt][1] * inv0));
    }
    if (tr1 < a.n_tok) {
      view_store(a.out, tr1, h, d, apply_gate(a.gate, tr1, h, d, o[nt][2] * inv1));
      view_store(a.out, tr1, h, d + 1, apply_gate(a.gate, tr1, h, d + 1, o[nt][3] * inv1));
    }
  }
}

}  // namespace hl
