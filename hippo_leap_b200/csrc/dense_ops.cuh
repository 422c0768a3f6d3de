// The small row-wise operators of a dense llama / qwen3 layer around the attention path
// (src/hippo_leap/backends/naive.nim): embedding lookup (:2976-3001), RMSNorm over the embedding
// dimension (rmsnormColsKernel :2802-2842), SiLU(gate) * up (siluMulKernel :2179-2197).  Activations are
// token-major here ([n_tok][dim]); the residual stream stays fp32, GEMM inputs are written as fp16.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "hl_device.cuh"

namespace hl {

// x[t][:] = float(table[token[t]][:])
__global__ void embedding_f16_kernel(const __half* __restrict__ table, const int32_t* __restrict__ tokens, int n_emb,
                                     int n_vocab, float* __restrict__ x) {
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= n_vocab ? n_vocab - 1 : tok);
  const __half2* src = reinterpret_cast<const __half2*>(table + static_cast<int64_t>(tok) * n_emb);
  float2* dst = reinterpret_cast<float2*>(x + static_cast<int64_t>(t) * n_emb);
  for (int i = threadIdx.x; i < n_emb / 2; i += blockDim.x) dst[i] = __half22float2(src[i]);
}

// out[t][:] = fp16( x[t][:] * (1 / sqrt(mean(x[t]^2) + eps)) * w[:] ); one block per token row
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                           int dim, float eps, __half* __restrict__ out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a projection queued behind may start loading its weights
  const float* xr = x + static_cast<int64_t>(blockIdx.x) * dim;
  const float inv = block_rms_inv_256(xr, dim, eps);
  __half* orow = out + static_cast<int64_t>(blockIdx.x) * dim;
  for (int i = threadIdx.x; i < dim; i += 256) orow[i] = __float2half_rn(xr[i] * inv * w[i]);
}

// h[t][f] = fp16( silu(gate) * up ), gate = gu[t][2f], up = gu[t][2f + 1]: the fp16 output of ONE GEMM whose weight
// rows interleave gate and up
__global__ void silu_mul_kernel(const __half* __restrict__ gu, int n_ffn, int64_t total, __half* __restrict__ h) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a projection queued behind may start loading its weights
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t t = idx / n_ffn, f = idx % n_ffn;
  const __half2 p = reinterpret_cast<const __half2*>(gu)[t * n_ffn + f];
  h[idx] = silu_mul_f16(__low2half(p), __high2half(p));
}

// The same, eight outputs per thread: two 16-byte loads of (gate, up) pairs, one 16-byte store.  (One output per thread
// -- a 4-byte load and a 2-byte store each -- ran at a quarter of the memory rate: 70 us for the 100 MB of a
// 2048 x 8192 activation.)  gu and h contiguous, 16-byte aligned, total a multiple of 8.
__global__ void silu_mul_vec8_kernel(const __half* __restrict__ gu, int64_t total8, __half* __restrict__ h) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 a = reinterpret_cast<const uint4*>(gu)[2 * i], b = reinterpret_cast<const uint4*>(gu)[2 * i + 1];
    const uint32_t in[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __half2 p0 = *reinterpret_cast<const __half2*>(&in[2 * k]), p1 = *reinterpret_cast<const __half2*>(&in[2 * k + 1]);
      const __half2 r = __halves2half2(silu_mul_f16(__low2half(p0), __high2half(p0)), silu_mul_f16(__low2half(p1), __high2half(p1)));
      o[k] = *reinterpret_cast<const uint32_t*>(&r);
    }
    reinterpret_cast<uint4*>(h)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace hl
