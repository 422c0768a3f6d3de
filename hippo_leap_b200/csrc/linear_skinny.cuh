// out[M, N] = A[M, K] . W[N, K]^T (+ residual) for 5 <= M <= 16 token rows (the kernel itself takes up to 64): the projection of a decode step over
// several sequences.  Like the single-row GEMV it is bound by reading W once, but with M rows the multiply-adds no
// longer fit the FMA pipe next to that stream (at M = 4 the scalar kernel already spends half its issue slots on
// them), so they go to the tensor cores through warp MMAs, with the token rows padded to 16 / 32 / 64.
//
//   block = 64 rows of W (one 8-row group per warp) x one split of K;  grid = (ceil(N / 64), splits)
//   * every lane's 16-byte loads of W (four or eight 32-wide K steps in flight, issued before anything else) ARE the B
//     fragments of two m16n8k16 MMAs: lane (g, t) holds W[n0 + g][k + 8t .. 8t + 7]; the first four halfs serve
//     MMA 0 (logical k 2t, 2t+1, 2t+8, 2t+9), the last four MMA 1.  The A fragments read the activations with the
//     same permutation of k, so each physical k is multiplied exactly once -- no shuffles, no shared-memory staging
//     of W.
//   * the block's slice of A, [M_pad][split length] fp16, sits in shared memory (row stride 64 bytes modulo 128
//     against bank conflicts) and is shared by the eight warps.
//   * splits > 1 (few rows of W): partial tiles go to a scratch buffer; the block of a row group that finishes
//     LAST (an arrival counter; nobody waits) adds the splits in index order -- the result does not depend on
//     scheduling -- applies the residual and stores.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "hl_device.cuh"
#include "linear_f16.cuh"

namespace hl {

struct SkinnyArgs {
  LinearArgs g;
  float* part;     // [splits][M][N] partial sums (splits > 1)
  int32_t* done;   // [ceil(N / 64)] arrival counters, zero between launches
  int32_t splits, kl;  // kl: K per split, multiple of 32
};

// MT: 16-row tiles of token rows (M <= 16 * MT).  kDepth: 32-wide K steps of W in flight per lane -- 8 covers a whole
// 256-wide split with one round of loads; 4 keeps the register count low enough for five blocks per SM on long splits.
template <int MT, int kDepth>
__global__ void __launch_bounds__(256) linear_skinny_kernel(SkinnyArgs p) {
  extern __shared__ __align__(16) uint8_t skinny_smem[];
  const LinearArgs& g = p.g;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t = lane & 3;
  const int kb = blockIdx.y * p.kl, ke = min(g.K, kb + p.kl);
  const int n_row = blockIdx.x * 64 + warp * 8 + gq;  // this lane's row of W
  const __half* wrow = g.w + static_cast<int64_t>(min(n_row, g.N - 1)) * g.ldw;
  // shared-memory row stride in halfs: 64 bytes modulo 128, so that the two rows an 8-lane phase of a 16-byte load
  // touches fall into different banks
  const int lda_s = p.kl + ((p.kl & 63) == 0 ? 32 : 0);
  __half* a_s = reinterpret_cast<__half*>(skinny_smem);

  uint4 wreg[kDepth];
  const int k_lane = kb + 8 * t;
#pragma unroll
  for (int d = 0; d < kDepth; ++d) {
    const int k = k_lane + 32 * d;
    wreg[d] = k < ke ? __ldcs(reinterpret_cast<const uint4*>(wrow + k)) : make_uint4(0, 0, 0, 0);
  }
  // activations of this split -> shared memory; rows >= M and columns >= K are zero
  {
    const int chunks = p.kl >> 3;  // 16-byte chunks per row
    for (int idx = tid; idx < MT * 16 * chunks; idx += 256) {
      const int m = idx / chunks, c = idx - m * chunks, k = kb + 8 * c;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < g.M && k < ke) {
        const __half* src = g.a + static_cast<int64_t>(m) * g.lda + k;
        if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
          v = *reinterpret_cast<const uint4*>(src);
        } else {
          __half tmp[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) tmp[i] = src[i];
          v = *reinterpret_cast<const uint4*>(tmp);
        }
      }
      *reinterpret_cast<uint4*>(a_s + static_cast<size_t>(m) * lda_s + 8 * c) = v;
    }
  }
  __syncthreads();

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
  // the loop bounds are the same for every lane (the MMAs are warp-wide); a lane whose 8 columns lie past the end
  // of K multiplies zeros
  for (int k0 = kb; k0 < ke; k0 += 32 * kDepth) {
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      if (k0 + 32 * d < ke) {
        const int k = k0 + 32 * d + 8 * t;
        const uint4 w = wreg[d];
        const int kn = k + 32 * kDepth;  // refill this slot with the step kDepth ahead
        wreg[d] = kn < ke ? __ldcs(reinterpret_cast<const uint4*>(wrow + kn)) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const __half* ap = a_s + static_cast<size_t>(mt * 16 + gq) * lda_s + (k - kb);
          const uint4 lo = *reinterpret_cast<const uint4*>(ap);
          const uint4 hi = *reinterpret_cast<const uint4*>(ap + 8 * lda_s);
          const uint32_t a0[4] = {lo.x, hi.x, lo.y, hi.y}, a1[4] = {lo.z, hi.z, lo.w, hi.w};
          mma16816(acc[mt], a0, w.x, w.y);
          mma16816(acc[mt], a1, w.z, w.w);
        }
      }
    }
  }

  // D fragment: rows mt * 16 + gq (+ 8), columns n_base + 2t, 2t + 1
  const int n_base = blockIdx.x * 64 + warp * 8, n = n_base + 2 * t;
  auto finish = [&](int m, int nn, float v) {
    if (g.resid != nullptr) v += g.resid[static_cast<int64_t>(m) * g.ldr + nn];
    if (g.out_dtype == HL_DTYPE_F32)
      static_cast<float*>(g.out)[static_cast<int64_t>(m) * g.ldo + nn] = v;
    else
      static_cast<__half*>(g.out)[static_cast<int64_t>(m) * g.ldo + nn] = __float2half_rn(v);
  };
  if (p.splits == 1) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int m = mt * 16 + gq + (e >> 1) * 8, nn = n + (e & 1);
        if (m < g.M && nn < g.N) finish(m, nn, acc[mt][e]);
      }
    return;
  }
  float* mine = p.part + static_cast<int64_t>(blockIdx.y) * g.M * g.N;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int m = mt * 16 + gq + (e >> 1) * 8, nn = n + (e & 1);
      if (m < g.M && nn < g.N) mine[static_cast<int64_t>(m) * g.N + nn] = acc[mt][e];
    }
  __shared__ int is_last;
  __threadfence();  // this thread's partials are visible device-wide before the block is counted
  __syncthreads();
  if (tid == 0) {
    const int prev = atomicAdd(p.done + blockIdx.x, 1);
    is_last = prev == p.splits - 1;
    if (is_last) p.done[blockIdx.x] = 0;  // every split has arrived: re-arm for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int n0 = blockIdx.x * 64, cols = min(64, g.N - n0);
  for (int idx = tid; idx < g.M * cols; idx += 256) {
    const int m = idx / cols, nn = n0 + idx - m * cols;
    float v = 0.f;
    for (int s = 0; s < p.splits; ++s) v += __ldcg(p.part + (static_cast<int64_t>(s) * g.M + m) * g.N + nn);
    finish(m, nn, v);
  }
}

}  // namespace hl
