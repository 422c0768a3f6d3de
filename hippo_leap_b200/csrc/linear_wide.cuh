// out[M, N] = A[M, K] . W[N, K]^T (+ residual) for 2 <= M <= 128 token rows on tcgen05, with the roles of the two
// operands swapped: the tensor core computes out^T -- 128 rows of W are the M side of the MMA, the (padded) token
// rows its N side -- so a tile is 128 x M_pad, there are N / 128 of them however few token rows there are, and W is
// streamed through shared memory exactly once.  (The square-tile GEMM of linear_f16.cuh has N / 256 tiles of 128 x 256
// at these sizes: eight CTAs for the 2048-wide projections.)  Split-K spreads short N over all SMs.
//
//   CTA = (128 rows of W, one split of K): warp 0 TMA producer (W box 128 x 64, A box M_pad x 64, 128-byte swizzle,
//   ring of stages), warp 1 MMA issuer + TMEM owner (tcgen05.mma kind::f16 M128 N=M_pad K16), warps 2-5 epilogue:
//   thread r owns W row r = output column n0 + r, reads its M_pad accumulator columns from TMEM and stores
//   out[m][n0 + r] -- lanes are consecutive columns, so every store instruction writes 128 contiguous bytes.
//   splits > 1: partial tiles to scratch; splitk_reduce_kernel, launched behind this kernel, adds
//   them in index order and applies the residual.  (Letting the CTA of a tile that arrives last do the sum was tried first:
//   one CTA adding the partials of its tile is a chain of L2 round trips that took longer than the streaming.)
//   Every barrier wait is bounded; TMEM is freed on every path.
#pragma once
#include <cuda.h>

#include "attn_prefill_tc.cuh"
#include "linear_f16.cuh"

namespace hl {

struct WideArgs {
  LinearArgs g;
  float* part;    // [splits][M][N]
  int32_t splits, kl, m_pad;  // kl: K per split (multiple of 64); m_pad: token rows padded to a multiple of 16
};

// out[m][n] = sum_s part[s][m][n] (+ residual), splits added in index order; four consecutive n per thread.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, int splits, LinearArgs g) {
  // launched with programmatic stream serialisation behind the kernel that writes the partials: resident early, it
  // waits here for that whole grid; the kernel behind this one may in turn start its own weight loads now
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t quads_per_row = (g.N + 3) >> 2;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= quads_per_row * g.M) return;
  const int m = static_cast<int>(idx / quads_per_row), n = static_cast<int>(idx % quads_per_row) * 4;
  const int64_t mn = static_cast<int64_t>(g.M) * g.N, off = static_cast<int64_t>(m) * g.N + n;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (n + 3 < g.N && (g.N & 3) == 0) {
    for (int s0 = 0; s0 < splits; s0 += 4) {
      float4 q[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        q[i] = s0 + i < splits ? __ldcs(reinterpret_cast<const float4*>(part + (s0 + i) * mn + off)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[0] += q[i].x;
        v[1] += q[i].y;
        v[2] += q[i].z;
        v[3] += q[i].w;
      }
    }
  } else {
    for (int s = 0; s < splits; ++s)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (n + e < g.N) v[e] += part[s * mn + off + e];
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    if (n + e >= g.N) break;
    float x = v[e];
    if (g.resid != nullptr) x += g.resid[static_cast<int64_t>(m) * g.ldr + n + e];
    if (g.out_dtype == HL_DTYPE_F32)
      static_cast<float*>(g.out)[static_cast<int64_t>(m) * g.ldo + n + e] = x;
    else
      static_cast<__half*>(g.out)[static_cast<int64_t>(m) * g.ldo + n + e] = __float2half_rn(x);
  }
}

struct LinearWideCfg {
  static constexpr int BW = 128, BK = 64, kStages = 3;  // 96 KiB of stages: two CTAs per SM
  static constexpr int kWBytes = BW * BK * 2;  // 16 KiB
  static constexpr int kABytesMax = 128 * BK * 2;
  static constexpr int kStageBytes = kWBytes + kABytesMax;
  static constexpr int kBarOff = kStages * kStageBytes;
  static constexpr int kNumBars = 2 * kStages + 1;
  static constexpr int kSmemBytes = 1024 + kBarOff + kNumBars * 8 + 16;
  static constexpr int kThreads = 192;
};

__global__ void __launch_bounds__(192, 2)
    linear_wide_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap a_map, WideArgs p) {
  using Cfg = LinearWideCfg;
  constexpr int S = Cfg::kStages;
  const LinearArgs& g = p.g;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + Cfg::kBarOff);
  uint64_t* full = bars;
  uint64_t* empty = bars + S;
  uint64_t* acc_full = bars + 2 * S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // Launched with programmatic stream serialisation: this grid may become resident while the kernel in front of it
  // is still running.  W is written by no kernel, so the producer streams its first stages at once; everything that
  // reads or writes activations (the A loads, the epilogue) first waits for the grids in front (griddepcontrol.wait).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * Cfg::BW;
  const int kb = blockIdx.y * p.kl, ke = min(g.K, kb + p.kl);
  const int n_kb = (ke - kb + Cfg::BK - 1) / Cfg::BK;
  const uint32_t tmem_cols = p.m_pad <= 32 ? 32u : (p.m_pad <= 64 ? 64u : 128u);
  const uint32_t a_bytes = static_cast<uint32_t>(p.m_pad) * Cfg::BK * 2;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    // Read before griddepcontrol.wait on purpose: an earlier grid may still be running and may yet set the status
    // word, so this only catches failures that are already visible.  Missing a late one is harmless -- the flag only
    // shortens this CTA's own bounded waits -- and the host still reads the status word after the stream drains.
    *abort_flag = (g.status != nullptr && *g.status != 0) ? 1 : 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&w_map);
      tma_prefetch_desc(&a_map);
      const int n_first = n_kb < S ? n_kb : S;
      for (int it = 0; it < n_first; ++it) {  // W of the first stages, before the grid dependency is resolved
        mbar_arrive_expect_tx(&full[it], Cfg::kWBytes + a_bytes);
        tma_load_2d(base + it * Cfg::kStageBytes, &w_map, &full[it], kb + it * Cfg::BK, n0);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int it = 0; it < n_first; ++it)
        tma_load_2d(base + it * Cfg::kStageBytes + Cfg::kWBytes, &a_map, &full[it], kb + it * Cfg::BK, 0);
      for (int it = S; it < n_kb; ++it) {
        const int s = it % S;
        tc_wait(&empty[s], ((it / S) - 1) & 1, g.status, 780 + s, abort_flag);
        mbar_arrive_expect_tx(&full[s], Cfg::kWBytes + a_bytes);
        const uint32_t dst = base + s * Cfg::kStageBytes;
        tma_load_2d(dst, &w_map, &full[s], kb + it * Cfg::BK, n0);
        tma_load_2d(dst + Cfg::kWBytes, &a_map, &full[s], kb + it * Cfg::BK, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(128, p.m_pad, 0);
      for (int it = 0; it < n_kb; ++it) {
        const int s = it % S;
        tc_wait(&full[s], (it / S) & 1, g.status, 790 + s, abort_flag);
        tc_fence_after();
        const uint32_t sw = base + s * Cfg::kStageBytes, sa = sw + Cfg::kWBytes;
#pragma unroll
        for (int ks = 0; ks < Cfg::BK / 16; ++ks)
          tc_mma_ss(tmem, umma_desc(sw + ks * 32, 16, 1024), umma_desc(sa + ks * 32, 16, 1024), idesc,
                    (it > 0 || ks > 0) ? 1u : 0u);
        tc_commit(&empty[s]);
      }
      tc_commit(acc_full);
    }
    __syncwarp();
  } else {
    // ---- epilogue: TMEM lane = row of W = output column ----
    const int quad = warp & 3;
    const int n = n0 + quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the residual / output buffers belong to earlier kernels until now
    tc_wait(acc_full, 0, g.status, 795, abort_flag);
    tc_fence_after();
    float* mine = p.splits > 1 ? p.part + static_cast<int64_t>(blockIdx.y) * g.M * g.N : nullptr;
    for (int c0 = 0; c0 < p.m_pad; c0 += 32) {
      float v[32];
      tc_ld32f(tmem + lane_sel + c0, v);  // columns past m_pad (m_pad = 16, 48, ...) are never stored
      tc_wait_ld();
      if (n < g.N) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int m = c0 + i;
          if (m < g.M) {
            if (mine != nullptr) {
              mine[static_cast<int64_t>(m) * g.N + n] = v[i];
            } else {
              float x = v[i];
              if (g.resid != nullptr) x += g.resid[static_cast<int64_t>(m) * g.ldr + n];
              if (g.out_dtype == HL_DTYPE_F32)
                static_cast<float*>(g.out)[static_cast<int64_t>(m) * g.ldo + n] = x;
              else
                static_cast<__half*>(g.out)[static_cast<int64_t>(m) * g.ldo + n] = __float2half_rn(x);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
  }
}

}  // namespace hl
