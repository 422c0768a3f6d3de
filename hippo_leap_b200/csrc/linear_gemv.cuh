// Decode projection out[m][n] = sum_k a[m][k] w[n][k] (+ residual) for M <= 4 token rows: the weight matrix is read
// once from HBM, so the kernel is a bandwidth problem.  Replaces the decode branch of gpuLinearCol / the
// linearHippo GEMV (src/hippo_leap/backends/naive.nim:3466-3547) and, through its prologue modes, the separate
// rmsnormCols (:2802-2842) launch in front of it and the siluMul (:2179-2197) launch behind it.
//
//   * Each block first builds the M activation rows as fp16 in shared memory:
//       mode 0  copy of fp16 rows
//       mode 1  RMSNorm of fp32 rows:  fp16(x * inv_rms * norm_w)
//     with the same arithmetic, in the same order, as rmsnorm_rows_kernel, so that a decode step and a prefill of
//     the same token feed bit-identical inputs to their GEMV / GEMM.
//   * Optional SwiGLU epilogue for a weight matrix whose rows interleave gate and up (row 2f = gate_f, row 2f+1 =
//     up_f):  out[m][f] = fp16(silu(fp16(gate)) * fp16(up)) -- the values silu_mul_kernel computes from the fp16
//     GEMM output in the prefill path.
//   * A warp owns R consecutive output rows and one of KS slices of K: per 256-wide step a lane has R independent
//     16-byte weight loads in flight against one shared-memory read of the activations.
//   * Launched with programmatic stream serialisation: a block first asks L2 to prefetch its weight rows
//     (which no kernel writes), lets the next kernel in the stream start, and only then waits for the kernels before
//     it (griddepcontrol.wait) and reads activations.  A chain of these keeps HBM busy across kernel boundaries.
//   * KS > 1 (few output rows): the KS slice warps of a row group sit in one block; partial sums meet in shared
//     memory and are added in slice order, so the result does not depend on scheduling.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "hl_device.cuh"
#include "linear_f16.cuh"

namespace hl {

enum : int32_t { kGemvPlain = 0, kGemvRmsNorm = 1 };

struct GemvArgs {
  LinearArgs g;          // a: fp16 rows (mode 0); out: [M][ldo], N columns, or N / 2 fp16 columns with the SwiGLU epilogue
  const float* x;        // mode 1: fp32 rows [M][ldx]
  const float* norm_w;   // mode 1: [K]
  int64_t ldx;
  float eps;
  int32_t mode, swiglu, ks, kslice;  // kslice: multiple of 256
};

template <int MAXM, int R>
__global__ void __launch_bounds__(256, MAXM == 1 ? 4 : 2) linear_gemv_fused_kernel(GemvArgs p) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  const LinearArgs& g = p.g;
  const int K = g.K, M = g.M;
  __half* a_s = reinterpret_cast<__half*>(gemv_smem);                        // [M][K]
  float* part = reinterpret_cast<float*>(gemv_smem + static_cast<size_t>(M) * K * 2);  // [8][MAXM][R]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int gw = blockIdx.x * 8 + warp;
  const int rg = gw / p.ks, ks = gw - rg * p.ks;
  const int n0 = rg * R;
  const bool live = n0 < g.N;
  const int kbeg = ks * p.kslice, kend = min(K, kbeg + p.kslice);
  // Weights only (no kernel writes them), so this is safe before the grid dependency is resolved: the first kDepth
  // 256-wide steps of the warp's rows go straight to registers, the rest of its slice is requested into L2.
  constexpr int kDepth = 2;
  const __half* wbase = g.w + static_cast<int64_t>(live ? n0 : 0) * g.ldw;  // rows past N - 1 re-read row N - 1
  const int ldw = static_cast<int>(g.ldw), rmax = g.N - 1 - n0;
#define HL_GEMV_WROW(r) (wbase + min((r), rmax) * ldw)
  const int k0 = kbeg + lane * 8;
  uint4 buf[kDepth][R];
  if (live) {
#pragma unroll
    for (int d = 0; d < kDepth; ++d)
      if (k0 + d * 256 < kend) {
#pragma unroll
        for (int r = 0; r < R; ++r) buf[d][r] = __ldcs(reinterpret_cast<const uint4*>(HL_GEMV_WROW(r) + k0 + d * 256));
      }
    const int pbeg = kbeg + kDepth * 256;
    if (lane < R && n0 + lane < g.N && kend > pbeg) {
      const __half* row = g.w + static_cast<int64_t>(n0 + lane) * g.ldw + pbeg;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(row), "r"((kend - pbeg) * 2) : "memory");
    }
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- prologue: activation rows -> shared memory (fp16)
  for (int m = 0; m < M; ++m) {
    __half* dst = a_s + static_cast<size_t>(m) * K;
    if (p.mode == kGemvRmsNorm) {
      const float* xr = p.x + m * p.ldx;
      const float inv = block_rms_inv_256(xr, K, p.eps);
      if (((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(p.norm_w)) & 15) == 0) {
        for (int i = tid * 4; i < K; i += 1024) {
          const float4 xv = *reinterpret_cast<const float4*>(xr + i);
          const float4 wv = *reinterpret_cast<const float4*>(p.norm_w + i);
          __half2 lo = __halves2half2(__float2half_rn(xv.x * inv * wv.x), __float2half_rn(xv.y * inv * wv.y));
          __half2 hi = __halves2half2(__float2half_rn(xv.z * inv * wv.z), __float2half_rn(xv.w * inv * wv.w));
          uint2 o;
          o.x = *reinterpret_cast<uint32_t*>(&lo);
          o.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(dst + i) = o;
        }
      } else {
        for (int i = tid; i < K; i += 256) dst[i] = __float2half_rn(xr[i] * inv * p.norm_w[i]);
      }
    } else {
      const __half* ar = g.a + m * g.lda;
      if ((reinterpret_cast<uintptr_t>(ar) & 15) == 0) {
        for (int i = tid * 8; i < K; i += 2048) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(ar + i);
      } else {
        for (int i = tid; i < K; i += 256) dst[i] = ar[i];
      }
    }
  }
  __syncthreads();

  float acc[MAXM][R];
#pragma unroll
  for (int m = 0; m < MAXM; ++m)
#pragma unroll
    for (int r = 0; r < R; ++r) acc[m][r] = 0.f;
  if (live) {
    for (int kb = k0; kb < kend; kb += 256 * kDepth) {
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        const int k = kb + d * 256;
        if (k < kend) {
#pragma unroll
          for (int m = 0; m < MAXM; ++m) {
            if (m < M) {
              const uint4 av = *reinterpret_cast<const uint4*>(a_s + static_cast<size_t>(m) * K + k);
              const __half2* a2 = reinterpret_cast<const __half2*>(&av);
#pragma unroll
              for (int r = 0; r < R; ++r) {
                const __half2* w2 = reinterpret_cast<const __half2*>(&buf[d][r]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 wf = __half22float2(w2[i]), af = __half22float2(a2[i]);
                  acc[m][r] = fmaf(wf.x, af.x, acc[m][r]);
                  acc[m][r] = fmaf(wf.y, af.y, acc[m][r]);
                }
              }
            }
          }
          const int kn = k + 256 * kDepth;  // refill this slot with the step kDepth ahead
          if (kn < kend) {
#pragma unroll
            for (int r = 0; r < R; ++r) buf[d][r] = __ldcs(reinterpret_cast<const uint4*>(HL_GEMV_WROW(r) + kn));
          }
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MAXM; ++m)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float v = acc[m][r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[m][r] = v;
    }
  if (p.ks > 1) {
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MAXM; ++m)
#pragma unroll
        for (int r = 0; r < R; ++r) part[(warp * MAXM + m) * R + r] = acc[m][r];
    }
    __syncthreads();
    if (ks != 0) return;
#pragma unroll
    for (int m = 0; m < MAXM; ++m)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float v = acc[m][r];
        for (int s = 1; s < p.ks; ++s) v += part[((warp + s) * MAXM + m) * R + r];
        acc[m][r] = v;
      }
  }
  if (!live || lane != 0) return;
#pragma unroll
  for (int m = 0; m < MAXM; ++m) {
    if (m >= M) break;
    if (p.swiglu) {
#pragma unroll
      for (int r = 0; r < R; r += 2) {
        const int n = n0 + r;
        if (n + 1 >= g.N) break;
        static_cast<__half*>(g.out)[m * g.ldo + (n >> 1)] =
            silu_mul_f16(__float2half_rn(acc[m][r]), __float2half_rn(acc[m][r + 1]));
      }
      continue;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int n = n0 + r;
      if (n >= g.N) break;
      float v = acc[m][r];
      if (g.resid != nullptr) v += g.resid[m * g.ldr + n];
      if (g.out_dtype == HL_DTYPE_F32)
        static_cast<float*>(g.out)[m * g.ldo + n] = v;
      else
        static_cast<__half*>(g.out)[m * g.ldo + n] = __float2half_rn(v);
    }
  }
}

#undef HL_GEMV_WROW

}  // namespace hl
