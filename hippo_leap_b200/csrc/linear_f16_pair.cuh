// out[M, N] = A[M, K] . W[N, K]^T (+ residual) on PAIRS of SMs: tcgen05.mma.cta_group::2, 256 x 256 output tiles.
//
// The single-SM GEMM (linear_f16.cuh) moves 48 KiB of operands from L2 into shared memory per 128 x 256 x 64 step,
// which at the tensor rate is more than the L2 -> SM path sustains on 148 SMs at once (its tensor pipe is busy 70 %
// of the time).  Here the two CTAs of a cluster compute one 256 x 256 tile: CTA r loads the A rows [128 r, +128)
// and the W rows (output columns) [128 r, +128) of every K step -- 32 KiB per SM instead of 48 -- and one thread of
// the leader CTA issues MMAs of M = 256, N = 256 that read A from both CTAs and the two halves of B from both
// shared memories; each CTA ends up with its 128 rows x 256 columns of the accumulator in its own TMEM.
//
//   per CTA: warp 0 TMA producer, warp 1 TMEM owner (+ MMA issuer in the leader), warps 2-5 epilogue
//   full[s]      leader only: posts the bytes of BOTH CTAs' loads; the peer's TMA completes on it (cta_group::2 form)
//   empty[s]     both CTAs, signalled by tcgen05.commit with a CTA mask
//   acc_full[b]  both CTAs, same
//   acc_empty[b] leader only, 256 arrivals: the epilogue threads of both CTAs (the peer's arrive through the cluster)
// Six stages, two accumulators of 256 columns.  No TMA multicast.  Every wait is bounded; TMEM is released on
// every path.  Used for M >= 512; smaller M keeps the single-SM kernel.
#pragma once
#include <cuda.h>

#include "attn_prefill_tc2.cuh"
#include "linear_f16.cuh"

namespace hl {

struct LinearPairCfg {
  static constexpr int BM = 128, BNH = 128, BK = 64, kStages = 6;  // per CTA: 128 rows of A, 128 rows of W
  static constexpr int kABytes = BM * BK * 2;   // 16 KiB
  static constexpr int kBBytes = BNH * BK * 2;  // 16 KiB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOff = kStages * kStageBytes;
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kSmemBytes = 1024 + kBarOff + kNumBars * 8 + 16;
  static constexpr int kThreads = 192;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
    linear_gemm_pair_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map,
                            LinearArgs g) {
  using Cfg = LinearPairCfg;
  constexpr int S = Cfg::kStages;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + Cfg::kBarOff);
  uint64_t* full = bars;
  uint64_t* empty = bars + S;
  uint64_t* acc_full = bars + 2 * S;       // [2]
  uint64_t* acc_empty = bars + 2 * S + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_m = (g.M + 255) / 256, tiles_n = (g.N + 255) / 256;
  const int n_tiles = tiles_m * tiles_n;
  const int n_kb = (g.K + Cfg::BK - 1) / Cfg::BK;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 256);
    }
    *abort_flag = (g.status != nullptr && *g.status != 0) ? 1 : 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anything can arrive on them
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs: own half of A rows and of W rows) ----------------
    if (lane == 0) {
      tma_prefetch_desc(&a_map);
      tma_prefetch_desc(&w_map);
      int it = 0;
      for (int tile = pair; tile < n_tiles; tile += n_pairs) {
        const int m0 = (tile % tiles_m) * 256 + 128 * static_cast<int>(rank);
        const int n0 = (tile / tiles_m) * 256 + 128 * static_cast<int>(rank);
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % S;
          if (it >= S) tc_wait(&empty[s], ((it / S) - 1) & 1, g.status, 740 + s, abort_flag);
          if (leader) mbar_arrive_expect_tx(&full[s], 2 * Cfg::kStageBytes);
          const uint32_t dst = base + s * Cfg::kStageBytes;
          tma2_load_2d(dst, &a_map, &full[s], kb * Cfg::BK, m0);
          tma2_load_2d(dst + Cfg::kABytes, &w_map, &full[s], kb * Cfg::BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc(256, 256, 0);
      int it = 0, ti = 0;
      for (int tile = pair; tile < n_tiles; tile += n_pairs, ++ti) {
        const int b = ti & 1;
        if (ti >= 2) tc_wait(&acc_empty[b], ((ti >> 1) - 1) & 1, g.status, 750 + b, abort_flag);
        tc_fence_after();
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % S;
          tc_wait(&full[s], (it / S) & 1, g.status, 760 + s, abort_flag);
          tc_fence_after();
          const uint32_t sa = base + s * Cfg::kStageBytes, sb = sa + Cfg::kABytes;
#pragma unroll
          for (int ks = 0; ks < Cfg::BK / 16; ++ks)
            tc2_mma_ss(tmem + b * 256, umma_desc(sa + ks * 32, 16, 1024), umma_desc(sb + ks * 32, 16, 1024), idesc,
                       (kb > 0 || ks > 0) ? 1u : 0u);
          tc2_commit_both(&empty[s]);
        }
        tc2_commit_both(&acc_full[b]);
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps (both CTAs): TMEM lane quadrant warp & 3, one output row per thread ----------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    int ti = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++ti) {
      const int b = ti & 1;
      const int m = (tile % tiles_m) * 256 + 128 * static_cast<int>(rank) + r;
      const int n0 = (tile / tiles_m) * 256;
      tc_wait(&acc_full[b], (ti >> 1) & 1, g.status, 770 + b, abort_flag);
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < 256; c0 += 32) {
        float v[32];
        tc_ld32f(tmem + lane_sel + b * 256 + c0, v);
        tc_wait_ld();
        const int n = n0 + c0;
        if (m < g.M && n < g.N) {
          const int nv = min(32, g.N - n);
          if (g.resid != nullptr) {
            // (scalar, predicated loads here -- 32 rows x 4 bytes per warp instruction -- cost 19 us of a 44 us
            // 2048 x 2048 x 2048 projection)
            const float* rp = g.resid + static_cast<int64_t>(m) * g.ldr + n;
            if (nv == 32 && (reinterpret_cast<uintptr_t>(rp) & 15) == 0) {
              float4 rr[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) rr[i] = reinterpret_cast<const float4*>(rp)[i];  // (plain loads: the residual may be the output buffer itself)
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                v[4 * i] += rr[i].x;
                v[4 * i + 1] += rr[i].y;
                v[4 * i + 2] += rr[i].z;
                v[4 * i + 3] += rr[i].w;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nv) v[i] += rp[i];
            }
          }
          if (g.out_dtype == HL_DTYPE_F32) {
            float* op = static_cast<float*>(g.out) + static_cast<int64_t>(m) * g.ldo + n;
            if (nv == 32 && (reinterpret_cast<uintptr_t>(op) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(op + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nv) op[i] = v[i];
            }
          } else if (g.out_dtype == kLinearOutSiluPairs) {
            store_silu_pairs32(g, m, n, nv, v);
          } else {
            __half* op = static_cast<__half*>(g.out) + static_cast<int64_t>(m) * g.ldo + n;
            if (nv == 32 && (reinterpret_cast<uintptr_t>(op) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 8)
                *reinterpret_cast<uint4*>(op + i) = make_uint4(pack_half2(v[i], v[i + 1]), pack_half2(v[i + 2], v[i + 3]),
                                                               pack_half2(v[i + 4], v[i + 5]), pack_half2(v[i + 6], v[i + 7]));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < nv) op[i] = __float2half_rn(v[i]);
            }
          }
        }
      }
      tc_fence_before();
      if (leader)
        mbar_arrive(&acc_empty[b]);
      else
        mbar_arrive_cluster(&acc_empty[b], 0);
    }
  }

  // ---- teardown: both CTAs are done with each other's shared memory and TMEM; release TMEM ----
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

}  // namespace hl
