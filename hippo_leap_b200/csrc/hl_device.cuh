// Device-side building blocks shared by the attention kernels (sm_100a only).
//
//  - mbarrier + TMA (cp.async.bulk.tensor, no multicast) wrappers with BOUNDED waits: a wait
//    that runs out records a status word in global memory and returns, so no kernel here can
//    spin for ever;
//  - the 128-byte shared-memory swizzle that TMA writes and ldmatrix / UMMA read;
//  - ldmatrix / mma.sync.m16n8k16 wrappers;
//  - the query prologue: raw Q row -> (RMSNorm) -> RoPE -> fp16, which replaces the reference's
//    qkNorm* and rope* kernels (src/hippo_leap/backends/naive.nim:2887-2971, 3006-3144).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hl_b200.h"

namespace hl {

// ---- device status word --------------------------------------------------------------
// status[0] = first error code (hl_status), status[1] = detail (where / which index).
__device__ __forceinline__ void report(int32_t* status, int32_t code, int32_t detail) {
  if (status && atomicCAS(status, 0, code) == 0) status[1] = detail;
}

// ---- shared-memory addressing ----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// A tile of rows of 128 bytes (64 halfs) written by TMA with CU_TENSOR_MAP_SWIZZLE_128B: the
// 16-byte chunk index is XOR-ed with the row index modulo 8.  `tile` must be 1024-byte aligned.
__device__ __forceinline__ uint32_t swz128(uint32_t tile, int row, int chunk) {
  return tile + row * 128 + (((chunk ^ row) & 7) << 4);
}

// ---- mbarrier ------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  try_wait itself suspends for a hardware time slice, so the limit below is of
// the order of a second, far beyond any legitimate wait in these kernels.  Returns false (after
// recording HL_ERR_TIMEOUT) when it gives up; callers carry on so that the grid still drains.
constexpr uint32_t kSpinLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int32_t* status,
                                          int32_t where) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  report(status, HL_ERR_TIMEOUT, where);
  return false;
}

// ---- TMA -----------------------------------------------------------------------------
// 2-D tiled load global -> this CTA's shared memory, completion counted on `bar`.
// c0 = innermost (element) coordinate: MUST be a multiple of 8 halfs (16 bytes).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint64_t* bar,
                                            int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ---- warp MMA --------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// 2^x for the softmax (x <= 0 there); the approximate unit is accurate to ~2^-22 relative.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void named_bar_sync(int id, int n_threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n_threads) : "memory");
}

// ---- strided activation views ------------------------------------------------------------
struct View {
  const void* ptr;
  int32_t dtype;
  int64_t ts, hs, ds;  // token, head, dim strides in elements
};
__device__ __forceinline__ float view_load(const View& v, int64_t t, int64_t h, int64_t d) {
  const int64_t off = t * v.ts + h * v.hs + d * v.ds;
  return v.dtype == HL_DTYPE_F16 ? __half2float(static_cast<const __half*>(v.ptr)[off])
                                 : static_cast<const float*>(v.ptr)[off];
}
__device__ __forceinline__ void view_store(const View& v, int64_t t, int64_t h, int64_t d,
                                           float x) {
  const int64_t off = t * v.ts + h * v.hs + d * v.ds;
  if (v.dtype == HL_DTYPE_F16)
    static_cast<__half*>(const_cast<void*>(v.ptr))[off] = __float2half_rn(x);
  else
    static_cast<float*>(const_cast<void*>(v.ptr))[off] = x;
}

// Optional output gate of the attention output: x * sigmoid(g), sigmoid(g) = 1 / (1 + expf(-g)), as
// attnGateKernel (src/hippo_leap/backends/naive.nim:2287-2293).  gate.ptr == nullptr means no gate.
__device__ __forceinline__ float apply_gate(const View& gate, int64_t t, int64_t h, int64_t d, float x) {
  if (gate.ptr == nullptr) return x;
  const float g = view_load(gate, t, h, d);
  return (1.0f / (1.0f + expf(-g))) * x;
}

// 1 / sqrt(mean(x^2) + eps) of one fp32 row, computed by a whole 256-thread block (every thread gets the value).
// One fixed order of additions: thread-strided partial sums, warp butterfly, eight warp sums added by index.
__device__ __forceinline__ float block_rms_inv_256(const float* __restrict__ xr, int dim, float eps) {
  __shared__ float red[8];
  __shared__ float inv_s;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += 256) ss += xr[i] * xr[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __syncthreads();  // a previous call's readers are done with red / inv_s
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < 8; ++i) tot += red[i];
    inv_s = 1.0f / sqrtf(tot / static_cast<float>(dim) + eps);
  }
  __syncthreads();
  return inv_s;
}

// fp16( silu(gate) * up ), silu(g) = g / (1 + expf(-g))   (siluMulKernel, naive.nim:2179-2197)
__device__ __forceinline__ __half silu_mul_f16(__half gate, __half up) {
  const float g = __half2float(gate), u = __half2float(up);
  const float sig = 1.0f / (1.0f + expf(-g));
  return __float2half_rn(g * sig * u);
}

// ---- row prologue: (RMSNorm) -> RoPE -------------------------------------------------------
// One WARP transforms one head row x[0..HD) held in shared memory as float32, in place.
//   norm : x <- x * (1/sqrt(mean(x^2) + eps)) * w        (naive.nim:2906-2917; tensor.nim:92-100)
//   rope : angle = float(pos) * theta[i], one fp32 multiply, then full-precision sincosf
//          (never the fast intrinsics: at position 32k a sloppy range reduction is visible)
//          pairs (2i, 2i+1) or (i, i+half)               (tensor.nim:156-166; naive.nim:3025-3030)
template <int HD>
__device__ __forceinline__ void norm_rope_row(float* x, const float* __restrict__ norm_w,
                                              float eps, const float* __restrict__ theta,
                                              int rope_dim, int rope_mode, int pos, int lane) {
  if (norm_w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int d = lane; d < HD; d += 32) ss += x[d] * x[d];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(HD) + eps);
#pragma unroll
    for (int d = lane; d < HD; d += 32) x[d] = x[d] * inv * norm_w[d];
    __syncwarp();
  }
  const int half = rope_dim >> 1;
  const float fpos = static_cast<float>(pos);
  for (int i = lane; i < half; i += 32) {
    const int i0 = rope_mode == HL_ROPE_INTERLEAVED ? 2 * i : i;
    const int i1 = rope_mode == HL_ROPE_INTERLEAVED ? 2 * i + 1 : i + half;
    const float angle = fpos * theta[i];
    float s, c;
    sincosf(angle, &s, &c);
    const float v0 = x[i0], v1 = x[i1];
    x[i0] = v0 * c - v1 * s;
    x[i1] = v0 * s + v1 * c;
  }
  __syncwarp();
}

// Write a float32 row (HD values in shared memory) as fp16 into a swizzled [rows][HD] tile made
// of HD/64 column-halves of `half_bytes` bytes each.  One warp per row.
template <int HD>
__device__ __forceinline__ void store_row_fp16_swz(uint32_t tile, int half_bytes, int row,
                                                   const float* x, int lane, bool zero) {
  // each lane writes pairs of halfs: HD/2 pairs over 32 lanes
#pragma unroll
  for (int p = lane; p < HD / 2; p += 32) {
    const int d = 2 * p;
    const uint32_t addr = swz128(tile + (d >> 6) * half_bytes, row, (d & 63) >> 3) + (d & 7) * 2;
    const uint32_t val = zero ? 0u : pack_half2(x[d], x[d + 1]);
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(val) : "memory");
  }
}

}  // namespace hl
