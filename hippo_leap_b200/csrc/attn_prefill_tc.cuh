// Causal GQA prefill on the 5th-generation tensor cores: tcgen05.mma with TMEM accumulators,
// TMA-staged K/V, fp32 online softmax with one thread per query row.
// Replaces qkNormPrefill(Q) + ropeAtPos(Q) + attentionPrefillKernel of the reference
// (src/hippo_leap/backends/naive.nim:2928-2971, 3006-3044, 3385-3464).
//
// One CTA = two 128-row tiles A and B that ping-pong on the tensor core: while the softmax warps of one tile
// work on S = Q K^T, the MMA warp runs the other tile.  The tiles are the SAME 128 query rows of two neighbouring
// query heads of one KV head (prompts of 768 to 16384 tokens, even group size: both tiles attend the same keys, so
// neither idles while the other finishes), or else two consecutive 128-row blocks of one head; either way they
// share every K / V tile.
//   warps 0-3  softmax of tile A  (thread r owns row r: TMEM lane r, no shuffles in the softmax)
//   warps 4-7  softmax of tile B
//   warp  8    TMA producer: K and V blocks of 128 keys from the paged cache, 128-byte swizzle; and, for
//              contiguous aligned query rows, ONE tiled load of the CTA's 256 raw rows into the idle K/V ring
//   warp  9    MMA issuer (one elected lane) and TMEM owner.  Inside the key loop it waits on no barrier (a
//              barrier wait costs this thread ~250 cycles while its MMAs are queued) and steps its descriptors with
//              one add per MMA (rebuilding them made the thread, not the tensor pipe, the bound)
//   warps 10-11  barrier scouts: wait on the K/V and P barriers in the issuer's order and publish step counters in
//              shared memory, which the issuer polls with acquire loads
// TMEM (512 columns): S_A, S_B (128 fp32 columns each; P, as fp16 pairs, overwrites the first 64
// columns of its S once the row has been read), O_A, O_B (head_dim columns each).
//   S_t  = Q_t K_j^T    tcgen05.mma kind::f16, A and B from shared memory (K-major, SW128)
//   O_t += P_t V_j      A from TMEM, B = V from shared memory as an MN-major SW128 operand
// The running maximum is only raised when it grows by more than 2^8 (the O rescale in TMEM then
// happens rarely); the final division by the row sum restores exactness.  After a tile's first block the
// exponentials therefore start at once against the running maximum, with the block's row maximum computed
// beside them; a row that does need a higher maximum has its first half done again.
// The query prologue (RMSNorm, RoPE from a cos/sin table built with full-precision sincosf, fp16)
// is done by the softmax warps while the first K/V blocks are in flight.
// Every wait is bounded; a timeout raises the status word, makes all later waits of the CTA fall
// through, and TMEM is always released before the CTA exits.
#pragma once
#include <cuda.h>

#include <type_traits>

#include "attn_prefill_mma.cuh"
#include "hl_device.cuh"
#include "host_common.h"

namespace hl {

struct PrefillTcArgs {
  PrefillArgs p;
  const float2* cs_table;  // [n_pos][rope_dim/2] (cos, sin) of float(pos) * theta_i
  int32_t box_rows;        // rows per TMA box: 16, or 128 when a block holds whole 128-key tiles
  uint32_t oob_row;        // a row coordinate outside the pool: TMA fills such boxes with zeros
  // Extra destinations of the output (same dtype and strides as p.out): peer GPUs' buffers mapped
  // into this GPU's address space.  The epilogue stores every tile to all of them with plain stores
  // over NVLink, so the all-gather of head outputs rides along with the compute.
  void* bcast[7];
  int32_t n_bcast;
  // 1: the raw query rows of the CTA are fetched by ONE tiled TMA load into the (still idle) K/V ring and the prologue
  // reads them from shared memory; needs contiguous, 16-byte aligned head rows (set by the launcher with the map).
  int32_t q_stage;
  int32_t early_q;  // 1: the query rows are known to be complete before this grid can start (read before the wait)
  // 1: the two tiles of a CTA are the SAME 128 query rows of two neighbouring heads of one KV head (heads 2x and 2x + 1;
  // the group size is even) instead of two consecutive 128-row blocks of one head.  Both tiles then attend exactly the
  // same keys: neither waits for the other at the end (the second row block always has one key block more: ~2 us per
  // CTA with the first tile's share of the SM idle), and they still share every K / V tile.
  int32_t pair_heads;
};

// 3-D tiled load global -> this CTA's shared memory (no multicast), completion counted on `bar`.
// c0 = innermost (element) coordinate: must be a multiple of 16 bytes (0 here).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint64_t* bar, int32_t c0, int32_t c1,
                                            int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// ---- tcgen05 wrappers --------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Lean forms for the issuing thread's inner loop.  A shared-memory matrix descriptor only varies in its low word (start
// address and leading byte offset, both in 16-byte units); the high word (stride byte offset, version, swizzle mode) is
// a constant of the layout.  Stepping an operand along K is then ONE 32-bit add per MMA: measured, building both
// descriptors from scratch for every MMA (~25 scalar instructions) made the single issuing thread, not the tensor
// pipe, the bound -- 85 cycles per 128x128x16 MMA against the 64 the pipe takes when fed.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}
__host__ __device__ constexpr uint32_t umma_desc_hi(uint32_t sbo_bytes) { return (sbo_bytes >> 4) | (1u << 14) | (2u << 29); }
__device__ __forceinline__ void tc_mma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(hi), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(hi), "r"(accumulate)
      : "memory");
}
#define HL_R32(a, o)                                                                                        \
  a[o + 0], a[o + 1], a[o + 2], a[o + 3], a[o + 4], a[o + 5], a[o + 6], a[o + 7], a[o + 8], a[o + 9],        \
      a[o + 10], a[o + 11], a[o + 12], a[o + 13], a[o + 14], a[o + 15], a[o + 16], a[o + 17], a[o + 18],    \
      a[o + 19], a[o + 20], a[o + 21], a[o + 22], a[o + 23], a[o + 24], a[o + 25], a[o + 26], a[o + 27],    \
      a[o + 28], a[o + 29], a[o + 30], a[o + 31]
// 32 consecutive TMEM columns of this thread's lane -> 32 registers
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld32f(uint32_t taddr, float* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31}, [%32];"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
        "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]),
        "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]),
        "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_st32f(uint32_t taddr, const float* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31,%32};" ::"r"(taddr),
      "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]), "f"(r[8]), "f"(r[9]),
      "f"(r[10]), "f"(r[11]), "f"(r[12]), "f"(r[13]), "f"(r[14]), "f"(r[15]), "f"(r[16]), "f"(r[17]), "f"(r[18]),
      "f"(r[19]), "f"(r[20]), "f"(r[21]), "f"(r[22]), "f"(r[23]), "f"(r[24]), "f"(r[25]), "f"(r[26]), "f"(r[27]),
      "f"(r[28]), "f"(r[29]), "f"(r[30]), "f"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Packed pairs of float32 (sm_100 has two-wide fp32 FMA / ADD): halves the issue slots of the
// scale-and-subtract and of the row sum in the softmax.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// VEC consecutive dims of one head row (dim stride 1), as one vector load when the address allows.
template <int VEC>
__device__ __forceinline__ void load_vec(const View& v, int64_t t, int64_t h, int d0, float* x) {
  const int64_t off = t * v.ts + h * v.hs + d0;
  if (v.dtype == HL_DTYPE_F32) {
    const float* p = static_cast<const float*>(v.ptr) + off;
    if ((reinterpret_cast<uintptr_t>(p) & (VEC * 4 - 1)) == 0) {
      if constexpr (VEC == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        x[0] = q.x; x[1] = q.y; x[2] = q.z; x[3] = q.w;
      } else {
        const float2 q = *reinterpret_cast<const float2*>(p);
        x[0] = q.x; x[1] = q.y;
      }
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) x[e] = p[e];
    }
  } else {
    const __half* p = static_cast<const __half*>(v.ptr) + off;
    if ((reinterpret_cast<uintptr_t>(p) & (VEC * 2 - 1)) == 0) {
      if constexpr (VEC == 4) {
        const uint2 q = *reinterpret_cast<const uint2*>(p);
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
        x[0] = lo.x; x[1] = lo.y; x[2] = hi.x; x[3] = hi.y;
      } else {
        const uint32_t q = *reinterpret_cast<const uint32_t*>(p);
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&q));
        x[0] = lo.x; x[1] = lo.y;
      }
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) x[e] = __half2float(p[e]);
    }
  }
}

// VEC consecutive dims of a raw row staged in shared memory (float32 or fp16), as one vector load.
template <int VEC>
__device__ __forceinline__ void load_vec_smem(uint32_t addr, bool f16, float* x) {
  if (!f16) {
    if constexpr (VEC == 4) {
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x[0]), "=f"(x[1]), "=f"(x[2]), "=f"(x[3]) : "r"(addr));
    } else {
      asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(x[0]), "=f"(x[1]) : "r"(addr));
    }
  } else {
    uint32_t lo, hi = 0;
    if constexpr (VEC == 4) {
      asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(addr));
    } else {
      asm volatile("ld.shared.b32 %0, [%1];" : "=r"(lo) : "r"(addr));
    }
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    x[0] = a.x;
    x[1] = a.y;
    if constexpr (VEC == 4) {
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
      x[2] = b.x;
      x[3] = b.y;
    }
  }
}

// 2^x for x <= 0 on the FMA / integer pipes (Cody-Waite split + degree-3 polynomial, relative error
// below 8e-5, far under the fp16 rounding P gets next).  A quarter of the softmax exponentials go
// through this instead of the special-function unit, which is the busiest unit of the kernel.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -126.0f);
  const float magic = 12582912.0f;  // 1.5 * 2^23: adding it leaves round(x) in the low mantissa bits
  const float xr = x + magic;
  const float f = x - (xr - magic);  // in [-0.5, 0.5]
  float p = fmaf(f, 0.05508868396282196f, 0.24260404706001282f);
  p = fmaf(p, f, 0.6932762265205383f);
  p = fmaf(p, f, 0.9999289512634277f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(xr) << 23));
}

// Shared-memory matrix descriptors (sm_100 format): start address, leading / stride byte offsets in
// 16-byte units, version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
         (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16: fp16 A and B, fp32 accumulator, M x N, B major selectable.
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N, int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

#ifndef HL_TC_POLY_MASK
#define HL_TC_POLY_MASK (-1)  // -1: every exponential on the special-function unit; 3: a quarter on the FMA pipe; 7: an eighth
#endif

template <int HD>
struct PrefillTcCfg {
  static constexpr int kStagesK = HD == 128 ? 3 : 4;  // K runs further ahead than V: Q K^T of block j+1 is issued
  static constexpr int kStagesV = HD == 128 ? 2 : 4;  // one P V earlier than V of block j+1 is needed
  static constexpr int kHalves = HD / 64;
  static constexpr int kHalfBytes = 128 * 128;              // 128 rows x 64 halfs
  static constexpr int kTileBytes = kHalves * kHalfBytes;   // one Q tile, one K block or one V block
  static constexpr int kQOff = 0;
  static constexpr int kKOff = 2 * kTileBytes;
  static constexpr int kVOff = kKOff + kStagesK * kTileBytes;
  // fp32 row staging of the general (slow) query prologue: 8 warps x one row.  It borrows the LAST V
  // stage, which the producer does not fill before the prologue has finished in that mode.
  static constexpr int kRowOff = kVOff + (kStagesV - 1) * kTileBytes;
  static constexpr int kBarOff = kVOff + kStagesV * kTileBytes;
  // Raw query rows (256 rows of head_dim floats or halfs) staged by bulk copies: every ring stage except K stage 0,
  // which takes the first K block meanwhile.  (fp32, head_dim 128: 128 KiB, exactly the four other stages.)
  static constexpr int kQRawOff = kKOff + kTileBytes;
  static constexpr int kQRawBytes = (kStagesK - 1 + kStagesV) * kTileBytes;
  static_assert(kQRawBytes >= 256 * HD * 4, "the ring must hold 256 raw float32 query rows");
  static constexpr int kNumBars = 2 * kStagesK + 2 * kStagesV + 8;
  static constexpr int kSmemBytes = 1024 + kBarOff + kNumBars * 8 + 32;  // + TMEM slot, abort flag, relay counters
  static constexpr int kThreads = 384;  // 12 warps: two softmax warpgroups + one warpgroup: TMA, MMA, two barrier scouts
  static constexpr int kTmemCols = 512;
  static constexpr uint32_t kColS = 0, kColO = 256;  // S_t at t*128, O_t at 256 + t*HD
};

// Bounded wait that also gives up at once when the CTA has already seen a timeout.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, int32_t* status, int32_t where,
                                        volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  report(status, HL_ERR_TIMEOUT, where);
  return false;
}

// Step counters relayed through shared memory from a scout thread (which waits on the barriers) to the MMA thread.
__device__ __forceinline__ void relay_publish(uint32_t* flag, uint32_t value) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(flag)), "r"(value) : "memory");
}
__device__ __forceinline__ bool relay_wait(uint32_t* flag, uint32_t need, int32_t* status, int32_t where,
                                           volatile int* abort_flag) {
  const uint32_t addr = smem_u32(flag);
  for (uint32_t i = 0; i < (kSpinLimit << 4); ++i) {  // a poll is a plain load: far shorter than a try_wait time slice
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    if (v >= need) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  report(status, HL_ERR_TIMEOUT, where);
  return false;
}

template <int HD>
__global__ void __launch_bounds__(384, 1)
    attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                           const __grid_constant__ CUtensorMap q_map, PrefillTcArgs ta) {
  using Cfg = PrefillTcCfg<HD>;
  constexpr int SK = Cfg::kStagesK, SV = Cfg::kStagesV;
  const PrefillArgs& a = ta.p;
  const bool fast_prologue = a.q.ds == 1 && a.rope_dim == HD && ta.cs_table != nullptr;
  const bool q_stage = fast_prologue && ta.q_stage != 0;
  // Heads vary fastest and query blocks run from the last (most keys) to the first, so the launch order is
  // longest-first over the WHOLE grid: the short blocks of every head fill the tail.  (With query blocks fastest the
  // last head's long blocks start last and run with most SMs idle: 0.71 ms instead of 0.64 ms at 8192 tokens when the order was chosen.)
  // Neighbouring CTAs are the query heads of one KV head, so they share K/V tiles in L2.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a kernel queued behind may begin its own set-up
  const int q_blk = gridDim.y - 1 - blockIdx.y;
  const int hstep = ta.pair_heads ? 1 : 0, tstep = ta.pair_heads ? 0 : 128;  // tile t: head h + hstep * t, rows from t0 + tstep * t
  const int h = ta.pair_heads ? 2 * blockIdx.x : blockIdx.x;
  const int kvh = h / a.group;
  const int t0 = q_blk * (ta.pair_heads ? 128 : 256);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + Cfg::kBarOff);
  uint64_t* k_full = bars;
  uint64_t* k_empty = bars + SK;
  uint64_t* v_full = bars + 2 * SK;
  uint64_t* v_empty = bars + 2 * SK + SV;
  uint64_t* s_full = bars + 2 * SK + 2 * SV;      // [2]
  uint64_t* p_full = bars + 2 * SK + 2 * SV + 2;  // [2]
  uint64_t* o_full = bars + 2 * SK + 2 * SV + 4;  // [2]
  uint64_t* q_ready = bars + 2 * SK + 2 * SV + 6;
  uint64_t* q_raw = bars + 2 * SK + 2 * SV + 7;  // raw query rows have landed in the ring (staged prologue)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // Relay counters: what the scout warps have seen complete, as step counts: [0] K/V operands, [1] / [2] P of tile A / B.
  uint32_t* relay = tmem_slot + 2;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // keys attended by tile t: [0, k_end[t]); 128-key blocks: n_blk[t]
  int k_end[2], n_blk[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int live = min(128, a.n_tok - (t0 + tstep * t));
    k_end[t] = live > 0 ? a.start_pos + t0 + tstep * t + live : 0;
    n_blk[t] = (k_end[t] + 127) >> 7;
  }
  const int n_max = max(n_blk[0], n_blk[1]);
  const int k_end_max = max(k_end[0], k_end[1]);

  if (tid == 0) {
    for (int s = 0; s < SK; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < SV; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&o_full[t], 1);
    }
    mbar_init(q_ready, 256);
    mbar_init(q_raw, 1);
    *abort_flag = (a.status != nullptr && *a.status != 0) ? 1 : 0;  // an earlier CTA already failed
    relay[0] = relay[1] = relay[2] = 0u;
    mbar_fence_init();
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(Cfg::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Register budget: 384 threads x 168 registers.  The TMA / MMA warpgroup gives most of its share to
  // the two softmax warpgroups, which hold a whole 128-column row of S per thread.
  // (setmaxnreg sits at the top of each role's branch so that the compiler sees which limit governs
  // which code.)
  if (warp == 8) {
    // ======================= TMA producer =======================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    if (!ta.early_q) asm volatile("griddepcontrol.wait;" ::: "memory");  // the query rows may come from the grid in front
    if (q_stage && lane == 0) {
      // The CTA's 256 raw query rows as ONE tiled load ({head_dim, 1 head, 256 tokens}, or {head_dim, 2 heads, 128
      // tokens} when the tiles are two heads: the launcher builds the map with the box; rows past the end of the
      // prompt are zero-filled) into the ring stages that stay idle until the prologue is over; the softmax warps read
      // them from shared memory.  (Through registers it took 32 loads per lane, ~4 us before the arithmetic could
      // start; one bulk copy per row was slower still: the copy engine's rate is per request, not per byte.)
      tma_prefetch_desc(&q_map);
      mbar_arrive_expect_tx(q_raw, 256u * HD * (a.q.dtype == HL_DTYPE_F16 ? 2u : 4u));
      tma_load_3d(base + Cfg::kQRawOff, &q_map, q_raw, 0, h, t0);
    }
    // Launched with programmatic stream serialisation this grid may start while the kernel in front -- the KV append of
    // the same prompt -- is still running: set-up and the query prologue do not depend on it, the cache does.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int boxes_per_half = 128 / ta.box_rows;           // 8 or 1
    const int n_boxes = boxes_per_half * Cfg::kHalves;      // per K (or V) block: <= 16
    const int box_bytes = ta.box_rows * 128;
    for (int j = 0; j < n_max; ++j) {
      const int sk = j % SK, sv = j % SV;
      // this lane's box of the block: which row group, which column half
      const int grp = lane / Cfg::kHalves, hh = lane % Cfg::kHalves;
      int row = static_cast<int>(ta.oob_row);
      if (lane < n_boxes) {
        const int tok = j * 128 + grp * ta.box_rows;
        if (tok < k_end_max) {
          const int lb = tok / a.block_tokens;
          int pb = lb < a.n_blocks_in_table ? a.block_table[lb] : -1;
          if (pb < 0 || pb >= a.num_blocks) {
            report(a.status, HL_ERR_BOUNDS, lb);
            pb = 0;
          }
          row = (pb * a.n_head_kv + kvh) * a.block_tokens + tok % a.block_tokens;
        }
      }
      const uint32_t dst_off = hh * Cfg::kHalfBytes + grp * box_bytes;
      // K block j
      if (j >= SK) tc_wait(&k_empty[sk], ((j / SK) - 1) & 1, a.status, 500 + sk, abort_flag);
      if (lane == 0) mbar_arrive_expect_tx(&k_full[sk], Cfg::kTileBytes);
      __syncwarp();
      if (lane < n_boxes)
        tma_load_2d(base + Cfg::kKOff + sk * Cfg::kTileBytes + dst_off, &k_map, &k_full[sk], hh * 64, row);
      // V block j
      if (j >= SV) tc_wait(&v_empty[sv], ((j / SV) - 1) & 1, a.status, 510 + sv, abort_flag);
      // the general query prologue stages its rows in the last V stage, the staged one in every stage but K stage 0:
      // keep out until it is done
      if ((!fast_prologue && j == SV - 1) || (q_stage && j == 0)) tc_wait(q_ready, 0, a.status, 515, abort_flag);
      if (lane == 0) mbar_arrive_expect_tx(&v_full[sv], Cfg::kTileBytes);
      __syncwarp();
      if (lane < n_boxes)
        tma_load_2d(base + Cfg::kVOff + sv * Cfg::kTileBytes + dst_off, &v_map, &v_full[sv], hh * 64, row);
      __syncwarp();
    }
  } else if (warp == 9) {
    // ======================= MMA issuer =======================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(128, 128, 0);
      constexpr uint32_t idesc_pv = umma_idesc(128, HD, 1);
      constexpr uint32_t kHi = umma_desc_hi(1024);  // every operand here: 8-row groups 1024 bytes apart, 128-byte swizzle
      const uint32_t q_lo0 = umma_desc_lo(base + Cfg::kQOff, 16);
      const uint32_t k_lo0 = umma_desc_lo(base + Cfg::kKOff, 16);
      const uint32_t v_lo0 = umma_desc_lo(base + Cfg::kVOff, Cfg::kHalfBytes);
      // S_t = Q_t K^T for the K block in stage `stage`
      auto issue_qk = [&](int t, int stage) {
        const uint32_t a_lo = q_lo0 + t * (Cfg::kTileBytes >> 4), b_lo = k_lo0 + stage * (Cfg::kTileBytes >> 4);
        const uint32_t d = tmem + Cfg::kColS + t * 128;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off16 = static_cast<uint32_t>(((ks >> 2) * Cfg::kHalfBytes + (ks & 3) * 32) >> 4);  // a constant
          tc_mma_ss_lo(d, a_lo + off16, b_lo + off16, kHi, idesc_qk, ks > 0 ? 1u : 0u);
        }
      };
      // O_t (+)= P_t V for the V block in stage `stage`; `first` clears the accumulator
      auto issue_pv = [&](int t, int stage, bool first) {
        const uint32_t b_lo = v_lo0 + stage * (Cfg::kTileBytes >> 4);
        const uint32_t d = tmem + Cfg::kColO + t * HD, p_tmem = tmem + Cfg::kColS + t * 128;
        tc_mma_ts_lo(d, p_tmem, b_lo, kHi, idesc_pv, first ? 0u : 1u);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks) tc_mma_ts_lo(d, p_tmem + ks * 8, b_lo + ks * (2048 >> 4), kHi, idesc_pv, 1u);
      };
      tc_wait(q_ready, 0, a.status, 520, abort_flag);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_after();
      if (n_max > 0) {
        tc_wait(&k_full[0], 0, a.status, 521, abort_flag);
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (n_blk[t] > 0) {
            issue_qk(t, 0);
            tc_commit(&s_full[t]);
          }
        tc_commit(&k_empty[0]);
      }
      int sk_next = SK > 1 ? 1 : 0, sv = 0;  // stage of K block j + 1, stage of V block j
      for (int j = 0; j < n_max; ++j) {
        bool next_qk = false;
        // Nothing in this loop waits on a barrier: for the thread that issues the MMAs a barrier wait is taken in order
        // behind the MMAs it has queued (~250 cycles measured even when the phase completed long ago; with six of them
        // per step the tensor pipe idled a third of the time).  The scout warps wait instead and publish step counts in
        // shared memory, which this thread reads with plain acquire loads.
        relay_wait(&relay[0], j + 1, a.status, 532, abort_flag);  // V of block j and K of block j + 1 have landed
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= n_blk[t]) continue;
          relay_wait(&relay[1 + t], j + 1, a.status, 530 + t, abort_flag);  // P of tile t, block j, is in TMEM
          tc_fence_after();
          issue_pv(t, sv, j == 0);
          if (j + 1 < n_blk[t]) {
            issue_qk(t, sk_next);
            tc_commit(&s_full[t]);
            next_qk = true;
          } else {
            tc_commit(&o_full[t]);
          }
        }
        tc_commit(&v_empty[sv]);
        if (next_qk) tc_commit(&k_empty[sk_next]);
        sv = sv + 1 == SV ? 0 : sv + 1;
        sk_next = sk_next + 1 == SK ? 0 : sk_next + 1;
      }
    }
    __syncwarp();
  } else if (warp >= 10) {
    // ======================= barrier scouts =======================
    // Warp 10 watches the K/V operand barriers and tile A's P barrier, warp 11 tile B's P barrier, in the order the
    // MMA warp needs them, and publish how far they got (release stores; the MMA thread's acquire loads pair with them,
    // so what the barrier ordered before the scout's wait -- TMA writes, the softmax threads' TMEM stores -- is ordered
    // before the MMA thread's next instruction too).
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (lane == 0) {
      const int t = warp - 10;
      for (int j = 0; j < n_max; ++j) {
        if (t == 0) {
          tc_wait(&v_full[j % SV], (j / SV) & 1, a.status, 560, abort_flag);
          if (j + 1 < n_max) tc_wait(&k_full[(j + 1) % SK], ((j + 1) / SK) & 1, a.status, 561, abort_flag);
          relay_publish(&relay[0], j + 1);
        }
        if (j < n_blk[t]) {
          tc_wait(&p_full[t], j & 1, a.status, 562 + t, abort_flag);
          relay_publish(&relay[1 + t], j + 1);
        }
      }
    }
    __syncwarp();
  } else {
    // ======================= softmax warps (tile t, row r) =======================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int t = warp >> 2;
    const int r = tid & 127;
    const int trow = t0 + tstep * t + r;        // token index of this thread's row
    const int ht = h + hstep * t;               // this tile's head
    const int pos = a.start_pos + trow;         // its position
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_sel + Cfg::kColS + t * 128;
    const uint32_t tO = tmem + lane_sel + Cfg::kColO + t * HD;

    // ---- Q prologue: this warp prepares rows [32*(warp&3), +32) of tile t ----
    if (!ta.early_q) asm volatile("griddepcontrol.wait;" ::: "memory");  // query rows, cos / sin table, norm weights
    {
      const uint32_t q_tile = base + Cfg::kQOff + t * Cfg::kTileBytes;
      constexpr int VEC = HD / 32;
      const bool fast = fast_prologue;
      float* xrow = reinterpret_cast<float*>(gen + Cfg::kRowOff) + warp * HD;
      if (fast) {
        // All 32 rows of the warp are requested before any arithmetic (one trip to HBM, not one per batch of rows),
        // and the cos / sin pairs are not loaded per row -- that would double the bytes -- but taken exactly from the
        // table every eighth row and advanced by one position per row with a complex multiply by (cos t, sin t) of
        // position 1: at most seven steps, ~1e-6 absolute drift, far inside the fp16 rounding of Q.
        constexpr int NA = VEC;  // angle slots per lane (interleaved pairing uses VEC / 2 of them)
        const int d0 = lane * VEC;
        const int last_pos = a.start_pos + a.n_tok - 1;
        const int row0 = (warp & 3) * 32;
        const int tt0 = t0 + tstep * t + row0;
        const bool inter = a.rope_mode == HL_ROPE_INTERLEAVED;
        float x[32][VEC];
        if (!q_stage) {
#pragma unroll
          for (int u = 0; u < 32; ++u) {
            if (tt0 + u < a.n_tok) {
              load_vec<VEC>(a.q, tt0 + u, ht, d0, x[u]);
            } else {
#pragma unroll
              for (int e = 0; e < VEC; ++e) x[u][e] = 0.f;
            }
          }
        }
        int ai[NA];
#pragma unroll
        for (int e = 0; e < NA; ++e) ai[e] = inter ? ((d0 >> 1) + (e < VEC / 2 ? e : 0)) : ((d0 + e) & (HD / 2 - 1));
        float2 step[NA], cs8[4][NA];
#pragma unroll
        for (int e = 0; e < NA; ++e) step[e] = ta.cs_table[(HD / 2) + ai[e]];  // position 1
#pragma unroll
        for (int b8 = 0; b8 < 4; ++b8) {
          const float2* csr = ta.cs_table + static_cast<int64_t>(min(a.start_pos + tt0 + 8 * b8, last_pos)) * (HD / 2);
#pragma unroll
          for (int e = 0; e < NA; ++e) cs8[b8][e] = csr[ai[e]];
        }
        float w[VEC];
        if (a.q_norm_w != nullptr) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) w[e] = a.q_norm_w[d0 + e];
        }
        if (q_stage) {
          // staged rows: the cos / sin and weight loads above are already on their way; now the bulk copies must have
          // landed.  A warp reads one row as 32 contiguous vectors (no bank conflicts).
          tc_wait(q_raw, 0, a.status, 545, abort_flag);
          const bool f16 = a.q.dtype == HL_DTYPE_F16;
          const uint32_t row_bytes = HD * (f16 ? 2u : 4u);
          // staged layout: [256 tokens][head_dim], or [128 tokens][2 heads][head_dim] when the tiles are two heads
          const uint32_t row_step = ta.pair_heads ? 2u * row_bytes : row_bytes;
          const uint32_t src0 = base + Cfg::kQRawOff + (ta.pair_heads ? (row0 * 2 + t) : (128 * t + row0)) * row_bytes +
                                d0 * (f16 ? 2u : 4u);
#pragma unroll
          for (int u = 0; u < 32; ++u) {
            if (tt0 + u < a.n_tok) {
              load_vec_smem<VEC>(src0 + u * row_step, f16, x[u]);
            } else {
#pragma unroll
              for (int e = 0; e < VEC; ++e) x[u][e] = 0.f;
            }
          }
        }
        // Two warps share a scheduler here, so latency is hidden by independent instructions of ONE warp: the rows
        // are worked on eight at a time (while the later rows are still on their way from memory), and every step
        // runs over the eight rows before the next dependent step starts.  1/sqrt is the hardware approximation
        // (2 ulp): the exact sqrtf + divide pair is a call with branches that serialises the rows (4 us per CTA),
        // and the result is rounded to fp16 a few lines further down.
#pragma unroll
        for (int b8 = 0; b8 < 4; ++b8) {
          if (a.q_norm_w != nullptr) {
            float ss[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              ss[k] = 0.f;
#pragma unroll
              for (int e = 0; e < VEC; ++e) ss[k] += x[8 * b8 + k][e] * x[8 * b8 + k][e];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
              for (int k = 0; k < 8; ++k) ss[k] += __shfl_xor_sync(0xffffffffu, ss[k], o);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float inv = rsqrtf(ss[k] * (1.0f / static_cast<float>(HD)) + a.eps);
#pragma unroll
              for (int e = 0; e < VEC; ++e) x[8 * b8 + k][e] = x[8 * b8 + k][e] * inv * w[e];
            }
          }
          float other[8][VEC];
          if (!inter) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
#pragma unroll
              for (int e = 0; e < VEC; ++e) other[k][e] = __shfl_xor_sync(0xffffffffu, x[8 * b8 + k][e], 16);
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int u = 8 * b8 + k;
            float2* cs = cs8[b8];  // row 0 of the group: exact table values; then one complex multiply per row
            if (k != 0) {
#pragma unroll
              for (int e = 0; e < NA; ++e) {
                const float2 c0 = cs[e];
                cs[e] = make_float2(c0.x * step[e].x - c0.y * step[e].y, c0.x * step[e].y + c0.y * step[e].x);
              }
            }
            if (inter) {
#pragma unroll
              for (int e = 0; e < VEC; e += 2) {
                const float2 c = cs[e >> 1];
                const float v0 = x[u][e], v1 = x[u][e + 1];
                x[u][e] = v0 * c.x - v1 * c.y;
                x[u][e + 1] = v0 * c.y + v1 * c.x;
              }
            } else {
#pragma unroll
              for (int e = 0; e < VEC; ++e) {
                const float2 c = cs[e];
                x[u][e] = (d0 + e < HD / 2) ? x[u][e] * c.x - other[k][e] * c.y : other[k][e] * c.y + x[u][e] * c.x;
              }
            }
            const int row = row0 + u;
            const uint32_t addr = swz128(q_tile + (d0 >> 6) * Cfg::kHalfBytes, row, (d0 & 63) >> 3) + (d0 & 7) * 2;
            if constexpr (VEC == 4) {
              asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(pack_half2(x[u][0], x[u][1])),
                           "r"(pack_half2(x[u][2], x[u][3]))
                           : "memory");
            } else {
              asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(pack_half2(x[u][0], x[u][1])) : "memory");
            }
          }
        }
      } else {
        for (int rr = 0; rr < 32; ++rr) {
          const int row = (warp & 3) * 32 + rr;
          const int tt = t0 + tstep * t + row;
          const bool live = tt < a.n_tok;
          if (live) {
#pragma unroll
            for (int d = lane; d < HD; d += 32) xrow[d] = view_load(a.q, tt, ht, d);
            __syncwarp();
            norm_rope_row<HD>(xrow, a.q_norm_w, a.eps, a.theta, a.rope_dim, a.rope_mode, a.start_pos + tt, lane);
          }
          store_row_fp16_swz<HD>(q_tile, Cfg::kHalfBytes, row, xrow, lane, !live);
          __syncwarp();
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(q_ready);
    }

    float m = -INFINITY, l = 0.f;
    const float c = a.scale_log2;
    // One key block of the online softmax.  `first` (a compile-time tag) is the tile's first block, whose row maximum
    // must be known before any exponential.  Every later block starts its exponentials at once against the RUNNING
    // maximum -- which is what they would be taken against anyway unless the row maximum grows by more than 2^8 -- and
    // computes the block's row maximum next to them (independent instruction streams in one basic block: the max
    // chain on the ALU, the exponentials on the special-function unit).  With the maximum first, its dependency chain
    // (~240 cycles, alone on its scheduler) sat in front of every block of the S -> P -> S chain that bounds the loop.
    // When a row does need a higher maximum (rare after the first blocks), the accumulator is rescaled and the first
    // half of the block is simply done again: S is still whole in TMEM because no P has been stored yet.
    auto softmax_block = [&](auto first_tag, int j) {
      constexpr bool first = decltype(first_tag)::value;
      float s[128];
      tc_wait(&s_full[t], j & 1, a.status, 540 + t, abort_flag);
      tc_fence_after();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) tc_ld32f(tS + q4 * 32, s + q4 * 32);
      tc_wait_ld();
      const int key0 = j * 128;
      const bool diag = key0 + 127 > a.start_pos + t0 + tstep * t;  // block touches this tile's diagonal
      if (diag) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (key0 + i > pos) s[i] = -INFINITY;
      }
      // row maximum: four independent chains of 3-input max
      auto row_max = [&]() {
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
        return fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]);
      };
      uint64_t sum2[4];  // four independent packed accumulators
      uint32_t pk[64];
      // 64 exponentials against the maximum m: P as fp16 pairs in pk, row sums in sum2
      auto exp_half = [&](auto half_tag) {
        constexpr int half_i = decltype(half_tag)::value;
        const float mc = m * c;
        const uint64_t c2 = pack_f32x2(c, c), nmc2 = pack_f32x2(-mc, -mc);
#pragma unroll
        for (int i = half_i * 64; i < half_i * 64 + 64; i += 2) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(s[i], s[i + 1]), c2, nmc2), x0, x1);
          const bool poly = HL_TC_POLY_MASK >= 0 && ((i >> 1) & HL_TC_POLY_MASK) == HL_TC_POLY_MASK;  // compile-time
          const float p0 = poly ? exp2_poly(x0) : fast_exp2(x0);
          const float p1 = poly ? exp2_poly(x1) : fast_exp2(x1);
          sum2[(i >> 1) & 3] = add_f32x2(sum2[(i >> 1) & 3], pack_f32x2(p0, p1));
          pk[i >> 1] = pack_half2(p0, p1);
        }
      };
      using Half0 = std::integral_constant<int, 0>;
      using Half1 = std::integral_constant<int, 1>;
      sum2[0] = sum2[1] = sum2[2] = sum2[3] = 0ull;  // bits of +0.0f pairs
      if constexpr (first) {
        m = row_max();
        exp_half(Half0{});
      } else {
        exp_half(Half0{});  // optimistic: against the running maximum
        const float mx = row_max();
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
          // the first half again, against the raised maximum (the whole warp: the TMEM load is warp-wide; rows that
          // kept their maximum get the same values as before)
          tc_ld32f(tS, s);
          tc_ld32f(tS + 32, s + 32);
          tc_wait_ld();
          if (diag) {
#pragma unroll
            for (int i = 0; i < 64; ++i)
              if (key0 + i > pos) s[i] = -INFINITY;
          }
          sum2[0] = sum2[1] = sum2[2] = sum2[3] = 0ull;
          exp_half(Half0{});
        }
      }
      tc_st32(tS, pk);  // the first half of P is on its way while the second is computed
      exp_half(Half1{});
      tc_st32(tS + 32, pk + 32);
      {
        float a0, a1;
        unpack_f32x2(add_f32x2(add_f32x2(sum2[0], sum2[1]), add_f32x2(sum2[2], sum2[3])), a0, a1);
        l += a0 + a1;
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[t]);
    };
    if (n_blk[t] > 0) softmax_block(std::true_type{}, 0);
    for (int j = 1; j < n_blk[t]; ++j) softmax_block(std::false_type{}, j);
    // ---- epilogue: O / l -> out ----
    asm volatile("griddepcontrol.wait;" ::: "memory");  // (satisfied long ago; orders the output stores behind the grid in front)
    if (n_blk[t] > 0) {
      tc_wait(&o_full[t], 0, a.status, 550 + t, abort_flag);
      tc_fence_after();
      const float inv = 1.0f / l;
      const bool live = trow < a.n_tok;
      // fp16 output with contiguous head rows goes through shared memory (this tile's Q area, idle now
      // that its last Q K^T has completed), so that whole 256-byte rows leave in coalesced 16-byte
      // lanes -- which matters most for the peer destinations, where a 16-byte store per row would
      // waste most of every NVLink packet.
      const bool staged = a.out.ds == 1 && a.out.dtype == HL_DTYPE_F16 && (a.out.ts & 7) == 0 && (a.out.hs & 7) == 0 &&
                          (reinterpret_cast<uintptr_t>(a.out.ptr) & 15) == 0;
      const uint32_t o_tile = base + Cfg::kQOff + t * Cfg::kTileBytes;  // [128 rows][HD halfs], 16-byte chunks XOR-swizzled
#pragma unroll
      for (int q4 = 0; q4 < HD / 32; ++q4) {
        float oreg[32];
        tc_ld32f(tO + q4 * 32, oreg);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) oreg[i] *= inv;
        if (live && a.gate.ptr != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i) oreg[i] = apply_gate(a.gate, trow, ht, q4 * 32 + i, oreg[i]);
        }
        if (staged) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            const int chunk = (q4 * 4 + (i >> 3)) ^ (r & (HD / 8 - 1));
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(o_tile + r * (HD * 2) + chunk * 16),
                         "r"(pack_half2(oreg[i], oreg[i + 1])), "r"(pack_half2(oreg[i + 2], oreg[i + 3])),
                         "r"(pack_half2(oreg[i + 4], oreg[i + 5])), "r"(pack_half2(oreg[i + 6], oreg[i + 7]))
                         : "memory");
          }
        } else if (live) {
          const int64_t off = static_cast<int64_t>(trow) * a.out.ts + static_cast<int64_t>(ht) * a.out.hs + q4 * 32;
          for (int dsti = 0; dsti <= ta.n_bcast; ++dsti) {  // destination 0 is the local output
            void* obase = dsti == 0 ? const_cast<void*>(a.out.ptr) : ta.bcast[dsti - 1];
            if (a.out.ds == 1 && a.out.dtype == HL_DTYPE_F16) {
              __half* dst = static_cast<__half*>(obase) + off;
#pragma unroll
              for (int i = 0; i < 32; i += 2) *reinterpret_cast<uint32_t*>(dst + i) = pack_half2(oreg[i], oreg[i + 1]);
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
              for (int i = 0; i < 32; ++i) view_store(ov, trow, ht, q4 * 32 + i, oreg[i]);
            }
          }
        }
      }
      if (staged) {
        named_bar_sync(1 + t, 128);  // the tile's 128 rows are in shared memory
        constexpr int kChunks = HD / 8;  // 16-byte chunks per row
        const int rows_live = min(128, a.n_tok - (t0 + tstep * t));
        for (int dsti = 0; dsti <= ta.n_bcast; ++dsti) {
          __half* obase = static_cast<__half*>(dsti == 0 ? const_cast<void*>(a.out.ptr) : ta.bcast[dsti - 1]) +
                          static_cast<int64_t>(ht) * a.out.hs;
          for (int idx = r; idx < rows_live * kChunks; idx += 128) {
            const int row = idx / kChunks, ch = idx % kChunks;
            uint4 val;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                         : "r"(o_tile + row * (HD * 2) + ((ch ^ (row & (kChunks - 1))) * 16)));
            *reinterpret_cast<uint4*>(obase + static_cast<int64_t>(t0 + tstep * t + row) * a.out.ts + ch * 8) = val;
          }
        }
      }
    }
  }

  // ---- teardown: everything issued has completed (or timed out); release TMEM ----
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::kTmemCols) : "memory");
  }
}

// cos/sin table for the query prologue: out[p][i] = (cos, sin)(float(p) * theta[i]), full-precision sincosf.
__global__ void rope_table_kernel(const float* __restrict__ theta, int half, int n_pos, float2* __restrict__ out) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(n_pos) * half) return;
  const int p = static_cast<int>(idx / half), i = static_cast<int>(idx % half);
  float s, c;
  sincosf(static_cast<float>(p) * theta[i], &s, &c);
  out[idx] = make_float2(c, s);
}

}  // namespace hl

// The tcgen05 kernel takes every shape the warp-MMA kernel takes except tiny problems, where launching
// 256-row CTAs wastes most of the tile.
inline bool hl_prefill_tc_supported(const hl::PrefillArgs& a, int head_dim) {
  return (head_dim == 64 || head_dim == 128) && a.n_tok >= 1;
}
inline bool hl_prefill_tc_default(const hl::PrefillArgs& a, int head_dim) {
  return hl_prefill_tc_supported(a, head_dim) && a.n_tok >= 256;
}

// Fills the kernel arguments shared by the tcgen05 prefill kernels: the cos/sin table up to the last position
// of this call (grow-only, rebuilt when theta changes), the out-of-bounds row, the broadcast destinations.
static int32_t hl_prefill_tc_fill_args(hl_ctx* ctx, hl_kv* kv, const hl::PrefillArgs& a, int head_dim,
                                       void* const* bcast, int n_bcast, hl::PrefillTcArgs* out) {
  using namespace hl;
  const int n_pos = a.start_pos + a.n_tok;
  const int half = a.rope_dim / 2;
  PrefillTcArgs& ta = *out;
  ta.p = a;
  ta.cs_table = nullptr;
  ta.n_bcast = n_bcast;
  ta.early_q = ctx->chain_pdl ? 1 : 0;
  for (int i = 0; i < n_bcast; ++i) ta.bcast[i] = bcast[i];
  if (a.rope_dim == head_dim) {
    if (ctx->cs_len < n_pos || ctx->cs_half != half) {
      HL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      if (ctx->cs_table) cudaFree(ctx->cs_table);
      ctx->cs_table = nullptr;
      ctx->cs_len = 0;
      ctx->scratch_epoch++;
      const int cap = ((n_pos + 4095) / 4096) * 4096;
      HL_CUDA(ctx, cudaMalloc(&ctx->cs_table, static_cast<size_t>(cap) * half * sizeof(float2)));
      const int64_t total = static_cast<int64_t>(cap) * half;
      rope_table_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, ctx->stream>>>(
          ctx->theta_d, half, cap, static_cast<float2*>(ctx->cs_table));
      ctx->launches++;
      HL_CUDA(ctx, cudaGetLastError());
      ctx->cs_len = cap;
      ctx->cs_half = half;
    }
    ta.cs_table = static_cast<const float2*>(ctx->cs_table);
  }
  ta.box_rows = 16;
  ta.oob_row = static_cast<uint32_t>(static_cast<uint64_t>(kv->num_blocks) * a.n_head_kv * kv->block_tokens);  // this layer's rows
  return HL_OK;
}

template <int HD>
static int32_t hl_launch_prefill_tc_t(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl::PrefillArgs& a,
                                      void* const* bcast, int n_bcast) {
  using namespace hl;
  using Cfg = PrefillTcCfg<HD>;
  auto kern = attn_prefill_tc_kernel<HD>;
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    HL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured[ctx->device & 15] = true;
  }
  PrefillTcArgs ta{};
  int32_t rc = hl_prefill_tc_fill_args(ctx, kv, a, HD, bcast, n_bcast, &ta);
  if (rc != HL_OK) return rc;
  const bool wide = kv->block_tokens % 128 == 0;
  ta.box_rows = wide ? 128 : 16;
  static const bool no_pair_heads = getenv("HL_B200_NO_PAIR_HEADS") != nullptr;  // for comparison runs
  // Measured on 32/8, 64/8 and 16/2 heads, head_dim 64 and 128: 2-6 % faster from 1024 to 6144 tokens (8 % at 64/8 heads
  // and 6144 tokens), even at 8192, 0.3 % slower at 32768 (the two-microsecond tail is nothing there), 0-3 % slower at
  // 512 -- where less than half a wave of CTAs runs and the longest CTA, now with both tiles busy to its end, is the
  // whole launch.
  ta.pair_heads = (a.group % 2 == 0 && a.n_tok >= 768 && a.n_tok <= 16384 && !no_pair_heads) ? 1 : 0;
  CUtensorMap q_map{};
  {
    // TMA staging of the raw query rows: contiguous head rows whose every start is 16-byte aligned, described by a
    // 3-D map {head_dim, heads, tokens} over the caller's view (any token / head stride order)
    const uint64_t el = a.q.dtype == HL_DTYPE_F16 ? 2 : 4;
    static const bool no_stage = getenv("HL_B200_NO_QSTAGE") != nullptr;
    ta.q_stage = !no_stage && a.q.ds == 1 && a.rope_dim == HD && reinterpret_cast<uintptr_t>(a.q.ptr) % 16 == 0 &&
                 a.q.ts > 0 && a.q.hs > 0 && (a.q.ts * el) % 16 == 0 && (a.q.hs * el) % 16 == 0;
    if (ta.q_stage) {
      typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
      cuuint64_t dims[3] = {static_cast<cuuint64_t>(HD), static_cast<cuuint64_t>(a.n_head), static_cast<cuuint64_t>(a.n_tok)};
      cuuint64_t strides[2] = {static_cast<cuuint64_t>(a.q.hs) * el, static_cast<cuuint64_t>(a.q.ts) * el};
      cuuint32_t box[3] = {static_cast<cuuint32_t>(HD), ta.pair_heads ? 2u : 1u, ta.pair_heads ? 128u : 256u};
      cuuint32_t estr[3] = {1, 1, 1};
      const CUresult r = reinterpret_cast<EncodeFn>(ctx->encode_tiled)(
          &q_map, a.q.dtype == HL_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
          const_cast<void*>(a.q.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) ta.q_stage = 0;  // a view the copy engine cannot describe: the register prologue takes it
    }
    if (!ta.q_stage) q_map = wide ? kv->k_map128[layer] : kv->k_map[layer];  // a valid map; never used by the kernel then
  }
  dim3 grid(ta.pair_heads ? a.n_head / 2 : a.n_head, ta.pair_heads ? (a.n_tok + 127) / 128 : (a.n_tok + 255) / 256);
  HL_CUDA(ctx, launch_pdl(kern, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, ctx->stream,
                          wide ? kv->k_map128[layer] : kv->k_map[layer], wide ? kv->v_map128[layer] : kv->v_map[layer],
                          q_map, ta));
  ctx->launches++;
  HL_CUDA(ctx, cudaGetLastError());
  return HL_OK;
}

inline int32_t hl_launch_prefill_tc(hl_ctx* ctx, hl_kv* kv, int32_t layer, const hl::PrefillArgs& a, int head_dim,
                                    void* const* bcast = nullptr, int n_bcast = 0) {
  return head_dim == 64 ? hl_launch_prefill_tc_t<64>(ctx, kv, layer, a, bcast, n_bcast)
                        : hl_launch_prefill_tc_t<128>(ctx, kv, layer, a, bcast, n_bcast);
}
