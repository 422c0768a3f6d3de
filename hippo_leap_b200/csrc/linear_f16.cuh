// out[M, N] = A[M, K] . W[N, K]^T (+ residual): the projections either side of attention, for fp16
// activations and weights with fp32 accumulation.  Replaces gpuLinearCol for dense weights
// (src/hippo_leap/backends/naive.nim:3466-3547: a 16x16-thread scalar GEMM for prefill and a
// 256-thread dot-product GEMV for decode) -- out[row, t] = sum_k W[row, k] x[k, t] there, the same
// contraction with tokens on the other axis.
//
// Prefill (M >= 16): persistent warp-specialised tcgen05 GEMM.
//   tile 128 x 256 x 64; TMA (128-byte swizzle) -> 4-stage shared-memory ring -> tcgen05.mma
//   kind::f16 M128 N256 K16 -> two 256-column TMEM accumulators, so the epilogue of tile i (four
//   warps, one output row per thread) overlaps the MMAs of tile i+1.
//   warp 0: TMA producer   warp 1: MMA issuer + TMEM owner   warps 2-5: epilogue
//   Ragged M / N / K edges: TMA zero-fills out-of-range boxes, the epilogue masks its stores.
// Decode (M < 16): weight-bandwidth-bound GEMV, one warp per output row, 16-byte loads of W,
//   the M activation rows reused from registers.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "attn_prefill_tc.cuh"

namespace hl {

struct LinearArgs {
  const __half* a;     // [M][lda]   (GEMV path; the GEMM path reads A through its tensor map)
  const __half* w;     // [N][ldw]
  void* out;           // [M][ldo] fp32 or fp16
  const float* resid;  // optional [M][ldr] fp32, added in the epilogue
  int64_t lda, ldw, ldo, ldr;
  int32_t M, N, K, out_dtype;
  int32_t* status;
};

// Internal value of LinearArgs::out_dtype (not part of the C ABI): fp16 output of N / 2 columns,
// out[m][c] = fp16(silu(fp16 acc[m][2c]) * fp16 acc[m][2c + 1]): W's rows interleave gate and up, so accumulator columns
// 2c and 2c + 1 are the two factors of output column c -- the value the separate row kernel computes from the fp16 GEMM
// output, written directly (half the bytes, one launch fewer).  Both tcgen05 GEMMs implement it.
constexpr int32_t kLinearOutSiluPairs = 100;

// Epilogue store of that form for 32 accumulator columns starting at even column n of row m.
__device__ __forceinline__ void store_silu_pairs32(const LinearArgs& g, int m, int n, int nv, const float (&v)[32]) {
  __half* op = static_cast<__half*>(g.out) + static_cast<int64_t>(m) * g.ldo + (n >> 1);
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const __half2 r = __halves2half2(silu_mul_f16(__float2half_rn(v[i]), __float2half_rn(v[i + 1])),
                                     silu_mul_f16(__float2half_rn(v[i + 2]), __float2half_rn(v[i + 3])));
    o[i >> 2] = *reinterpret_cast<const uint32_t*>(&r);
  }
  if (nv == 32 && (reinterpret_cast<uintptr_t>(op) & 15) == 0) {
    *reinterpret_cast<uint4*>(op) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(op + 8) = make_uint4(o[4], o[5], o[6], o[7]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (2 * i + 1 < nv) op[i] = __ushort_as_half(static_cast<unsigned short>(o[i >> 1] >> ((i & 1) * 16)));
  }
}

struct LinearGemmCfg {
  static constexpr int BM = 128, BN = 256, BK = 64, kStages = 4;
  static constexpr int kABytes = BM * BK * 2;  // 16 KiB
  static constexpr int kBBytes = BN * BK * 2;  // 32 KiB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOff = kStages * kStageBytes;
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kSmemBytes = 1024 + kBarOff + kNumBars * 8 + 16;
  static constexpr int kThreads = 192;
};

__global__ void __launch_bounds__(192, 1)
    linear_gemm_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map,
                       LinearArgs g) {
  using Cfg = LinearGemmCfg;
  constexpr int S = Cfg::kStages;
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
  const int tiles_m = (g.M + Cfg::BM - 1) / Cfg::BM, tiles_n = (g.N + Cfg::BN - 1) / Cfg::BN;
  const int n_tiles = tiles_m * tiles_n;
  const int n_kb = (g.K + Cfg::BK - 1) / Cfg::BK;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
    }
    *abort_flag = (g.status != nullptr && *g.status != 0) ? 1 : 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&a_map);
      tma_prefetch_desc(&w_map);
      int it = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * Cfg::BM, n0 = (tile / tiles_m) * Cfg::BN;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % S;
          if (it >= S) tc_wait(&empty[s], ((it / S) - 1) & 1, g.status, 700 + s, abort_flag);
          mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
          const uint32_t dst = base + s * Cfg::kStageBytes;
          tma_load_2d(dst, &a_map, &full[s], kb * Cfg::BK, m0);
          tma_load_2d(dst + Cfg::kABytes, &w_map, &full[s], kb * Cfg::BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(Cfg::BM, Cfg::BN, 0);
      int it = 0, ti = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
        const int b = ti & 1;
        if (ti >= 2) tc_wait(&acc_empty[b], ((ti >> 1) - 1) & 1, g.status, 710 + b, abort_flag);
        tc_fence_after();
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = it % S;
          tc_wait(&full[s], (it / S) & 1, g.status, 720 + s, abort_flag);
          tc_fence_after();
          const uint32_t sa = base + s * Cfg::kStageBytes, sb = sa + Cfg::kABytes;
#pragma unroll
          for (int ks = 0; ks < Cfg::BK / 16; ++ks)
            tc_mma_ss(tmem + b * 256, umma_desc(sa + ks * 32, 16, 1024), umma_desc(sb + ks * 32, 16, 1024), idesc,
                      (kb > 0 || ks > 0) ? 1u : 0u);
          tc_commit(&empty[s]);
        }
        tc_commit(&acc_full[b]);
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps: TMEM lane quadrant warp & 3, one output row per thread ----------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    int ti = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
      const int b = ti & 1;
      const int m0 = (tile % tiles_m) * Cfg::BM, n0 = (tile / tiles_m) * Cfg::BN;
      tc_wait(&acc_full[b], (ti >> 1) & 1, g.status, 730 + b, abort_flag);
      tc_fence_after();
      const int m = m0 + r;
#pragma unroll 1
      for (int c0 = 0; c0 < Cfg::BN; c0 += 32) {
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
      mbar_arrive(&acc_empty[b]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// Decode: out[m][n] = sum_k a[m][k] w[n][k] (+ resid), M <= 16.  One warp per output row n.
template <int MAXM>
__global__ void __launch_bounds__(256) linear_gemv_kernel(LinearArgs g) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= g.N) return;
  const __half* wrow = g.w + static_cast<int64_t>(warp) * g.ldw;
  float acc[MAXM];
#pragma unroll
  for (int m = 0; m < MAXM; ++m) acc[m] = 0.f;
  const bool vec = (g.K & 7) == 0 && (reinterpret_cast<uintptr_t>(wrow) & 15) == 0 && (g.lda & 7) == 0 &&
                   (reinterpret_cast<uintptr_t>(g.a) & 15) == 0;
  if (vec) {
    for (int k = lane * 8; k < g.K; k += 256) {
      const uint4 wv = *reinterpret_cast<const uint4*>(wrow + k);
      const __half2* w2 = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
      for (int m = 0; m < MAXM; ++m) {
        if (m < g.M) {
          const uint4 av = *reinterpret_cast<const uint4*>(g.a + static_cast<int64_t>(m) * g.lda + k);
          const __half2* a2 = reinterpret_cast<const __half2*>(&av);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 wf = __half22float2(w2[i]), af = __half22float2(a2[i]);
            acc[m] = fmaf(wf.x, af.x, acc[m]);
            acc[m] = fmaf(wf.y, af.y, acc[m]);
          }
        }
      }
    }
  } else {
    for (int k = lane; k < g.K; k += 32) {
      const float wf = __half2float(wrow[k]);
#pragma unroll
      for (int m = 0; m < MAXM; ++m)
        if (m < g.M) acc[m] = fmaf(wf, __half2float(g.a[static_cast<int64_t>(m) * g.lda + k]), acc[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < MAXM; ++m) {
    float v = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && m < g.M) {
      if (g.resid != nullptr) v += g.resid[static_cast<int64_t>(m) * g.ldr + warp];
      if (g.out_dtype == HL_DTYPE_F32)
        static_cast<float*>(g.out)[static_cast<int64_t>(m) * g.ldo + warp] = v;
      else
        static_cast<__half*>(g.out)[static_cast<int64_t>(m) * g.ldo + warp] = __float2half_rn(v);
    }
  }
}

}  // namespace hl
