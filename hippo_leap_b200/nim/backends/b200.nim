## B200 (sm_100a) backend for hippo_leap: the seven procs of the backend contract, bound to
## libhl_b200.so through its C ABI (include/hl_backend.h, include/hl_b200.h).
##
## Drop this file at src/hippo_leap/backends/b200.nim and add to src/hippo_leap/inference.nim,
## next to the existing arms (inference.nim:7-14):
##
##   elif defined(backendB200):
##     import ./backends/b200
##     export b200
##
## Build: nim cpp -d:backendB200 -d:HippoRuntime:CUDA --passL:"-lhl_b200 -lcudart" ...
##
## Scope: dense llama / qwen3 models whose weights can be held as fp16 (an F16 GGUF is exact; a quantised
## one is dequantised by Model.getTensor and rounded): embedding, RMSNorm, the projections, SwiGLU and the
## vocabulary projection run inside the library around its attention path (hl_dense_* in
## include/hl_backend.h).  MoE / SSM layers (lkAttnMoe, lkSsm*) are not covered and are rejected at load.
## With -d:b200Standin the attention-only stand-in model of hl_backend_* is bound instead (its tables are
## read from tensors named "standin.*").  No Nim toolchain was available where this file was written: it
## is a thin transliteration of the Python mirrors (hippo_leap_b200/dense.py, backend.py), which ARE
## exercised on a GPU.

when not defined(cpp):
  {.error: "the b200 backend requires Nim's C++ backend. Build with `nim cpp`.".}

import
  std/[tables, sequtils],
  ../[model, tensor, backend_types]

const hlLib = "libhl_b200.so"

type
  HlHParams {.bycopy.} = object
    nVocab, nLayer, nHead, nHeadKv, headDim, ropeDim: int32
    ropeFreqBase, rmsEps: float32
    ropeMode, llama3Scaling: int32

  HlStandinWeights {.bycopy.} = object
    eq, ek, ev, wout, qNorm, kNorm: ptr float32

  HlKvCache {.bycopy.} = object
    curLen, maxLen, nHeadKv, headDim: int32
    gpuCache: pointer

  HlDenseHParams {.bycopy.} = object
    nVocab, nEmb, nLayer, nFfn, nHead, nHeadKv, headDim, ropeDim: int32
    ropeFreqBase, rmsEps: float32
    ropeMode, llama3Scaling: int32

  HlDenseWeights {.bycopy.} = object
    ## fp16 matrices [out][in], stacked over layers; float32 norm vectors (include/hl_backend.h)
    tokEmb: ptr uint16
    attnNorm: ptr float32
    wq, wk, wv, wo: ptr uint16
    qNorm, kNorm, ffnNorm: ptr float32
    wGate, wUp, wDown: ptr uint16
    outNorm: ptr float32
    wOut: ptr uint16

const
  HlRopeSplitHalf = 1'i32   # the pairing of every reference GPU kernel (naive.nim:3025-3030)

proc hl_backend_init_kv_cache(device: int32, hp: ptr HlHParams, maxLen: int32,
                              cache: ptr HlKvCache): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_backend_free_kv_cache(cache: ptr HlKvCache): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_backend_load_model(device: int32, hp: ptr HlHParams,
                           w: ptr HlStandinWeights): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_backend_unload_model(): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_backend_forward_prefill(tokens: ptr int32, n: int32, cache: ptr HlKvCache,
                                logits: ptr float32): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_backend_forward_decode(token: int32, cache: ptr HlKvCache,
                               logits: ptr float32): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_backend_forward_decode_token(token: int32, cache: ptr HlKvCache,
                                     next: ptr int32): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_backend_forward_decode_token_timed(token: int32, cache: ptr HlKvCache, next: ptr int32,
                                           gpuMs: ptr float32): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_backend_last_error(): cstring {.importc, cdecl, dynlib: hlLib.}
proc hl_dense_init_kv_cache(device: int32, hp: ptr HlDenseHParams, maxLen: int32,
                            cache: ptr HlKvCache): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_dense_free_kv_cache(cache: ptr HlKvCache): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_dense_load_model(device: int32, hp: ptr HlDenseHParams,
                         w: ptr HlDenseWeights): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_dense_unload_model(): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_dense_forward_prefill(tokens: ptr int32, n: int32, cache: ptr HlKvCache,
                              logits: ptr float32): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_dense_forward_decode(token: int32, cache: ptr HlKvCache,
                             logits: ptr float32): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_dense_forward_decode_token_timed(token: int32, cache: ptr HlKvCache, next: ptr int32,
                                         gpuMs: ptr float32): int32 {.importc, cdecl, dynlib: hlLib.}
proc hl_dense_last_error(): cstring {.importc, cdecl, dynlib: hlLib.}
proc hl_b200_kv_layer(kv: pointer, layer: int32, kPool, vPool: ptr pointer,
                      bytesEach: ptr csize_t): int32 {.importc, cdecl, dynlib: hlLib.}

var
  # One library-side cache per KvCache handed out by initKvCache, keyed by the device pointer of its layer-0 K pool
  # (KvCache has no spare field for a handle).  Each KvCache owns its own device pools, as in the reference
  # (initGpuKvCache, naive.nim:3552-3567); all of them are freed by unloadModelBackend.
  shimCaches: Table[pointer, HlKvCache]
  shimHp: HlHParams

proc check(rc: int32) =
  ## Errors bubble as exceptions (AGENTS.md:224-230); the text comes from the library.
  if rc != 0:
    let msg = when defined(b200Standin): $hl_backend_last_error() else: $hl_dense_last_error()
    if rc == 4: raise newException(IOError, msg)       # HL_ERR_CUDA
    raise newException(ValueError, msg)

proc toHl(hp: HParams): HlHParams =
  HlHParams(nVocab: hp.nVocab.int32, nLayer: hp.nLayer.int32, nHead: hp.nHead.int32,
            nHeadKv: hp.nHeadKv.int32, headDim: hp.headDim.int32, ropeDim: hp.ropeDim.int32,
            ropeFreqBase: hp.ropeFreqBase, rmsEps: hp.rmsEps,
            ropeMode: HlRopeSplitHalf, llama3Scaling: 0)

proc syncIn(cache: KvCache): ptr HlKvCache =
  ## The library-side cache behind `cache`, with the caller's curLen: callers reset cache.curLen themselves
  ## (inference.nim:58); honour it.
  if cache.gpuCache.k.len == 0 or cache.gpuCache.k[0].devicePtr notin shimCaches:
    raise newException(ValueError, "KvCache was not created by this backend's initKvCache")
  result = addr shimCaches[cache.gpuCache.k[0].devicePtr]
  result.curLen = cache.curLen.int32

proc syncOut(cache: var KvCache, shim: ptr HlKvCache) =
  cache.curLen = shim.curLen.int
  cache.gpuCache.curLen = shim.curLen.int          # naive.nim:4586-4587

proc toDense(hp: HParams): HlDenseHParams =
  HlDenseHParams(nVocab: hp.nVocab.int32, nEmb: hp.nEmb.int32, nLayer: hp.nLayer.int32, nFfn: hp.nFfn.int32,
                 nHead: hp.nHead.int32, nHeadKv: hp.nHeadKv.int32, headDim: hp.headDim.int32,
                 ropeDim: hp.ropeDim.int32, ropeFreqBase: hp.ropeFreqBase, rmsEps: hp.rmsEps,
                 ropeMode: HlRopeSplitHalf, llama3Scaling: 0)

var shimDenseHp: HlDenseHParams

proc initKvCache*(hp: HParams, maxLen: int): KvCache =
  var shimCache: HlKvCache
  when defined(b200Standin):
    shimHp = toHl(hp)
    check hl_backend_init_kv_cache(0, addr shimHp, maxLen.int32, addr shimCache)
  else:
    shimDenseHp = toDense(hp)
    check hl_dense_init_kv_cache(0, addr shimDenseHp, maxLen.int32, addr shimCache)
  result.maxLen = maxLen
  result.curLen = 0
  result.nHeadKv = hp.nHeadKv
  result.headDim = hp.headDim
  result.gpuCache.maxLen = maxLen
  result.gpuCache.nHeadKv = hp.nHeadKv
  result.gpuCache.headDim = hp.headDim
  result.gpuCache.k = newSeq[GpuTensor](hp.nLayer)
  result.gpuCache.v = newSeq[GpuTensor](hp.nLayer)
  const blockTokens = when defined(b200Standin): 16 else: 128   # tokens per page of the pool
  let numBlocks = (maxLen + blockTokens - 1) div blockTokens
  for layer in 0 ..< hp.nLayer:
    var kp, vp: pointer
    var bytes: csize_t
    check hl_b200_kv_layer(shimCache.gpuCache, layer.int32, addr kp, addr vp, addr bytes)
    # the layer's page pools: fp16 [numBlocks, nHeadKv, blockTokens, headDim]; `alloc` stays default because
    # the library owns the memory
    result.gpuCache.k[layer] = GpuTensor(devicePtr: kp, shape: @[numBlocks, hp.nHeadKv, blockTokens, hp.headDim],
                                         sizeBytes: bytes.int)
    result.gpuCache.v[layer] = GpuTensor(devicePtr: vp, shape: @[numBlocks, hp.nHeadKv, blockTokens, hp.headDim],
                                         sizeBytes: bytes.int)
  shimCaches[result.gpuCache.k[0].devicePtr] = shimCache

proc floatToHalfRne(f: float32): uint16 =
  ## float32 -> fp16 bit pattern, round to nearest even, subnormals kept: the rounding of the CUDA kernels
  ## (__float2half_rn) and of the tested Python mirror (numpy's astype(float16)).  quant.floatToHalf
  ## (quant.nim:98-107) truncates the mantissa and flushes subnormals to zero, which would give this build other
  ## weights than the ones the parity tests ran on.  Values that are exact in fp16 (an F16 GGUF) convert exactly.
  let bits = cast[uint32](f)
  let sign = uint16((bits shr 16) and 0x8000'u32)
  let a = bits and 0x7FFFFFFF'u32
  if a > 0x7F800000'u32: return sign or 0x7E00'u16            # NaN
  if a >= 0x47800000'u32: return sign or 0x7C00'u16           # >= 65536 (and inf): infinity
  if a >= 0x38800000'u32:                                     # normal half: |f| >= 2^-14
    var h = (((a shr 23) - 112'u32) shl 10) or ((a shr 13) and 0x3FF'u32)
    let rem = a and 0x1FFF'u32
    if rem > 0x1000'u32 or (rem == 0x1000'u32 and (h and 1'u32) == 1'u32): inc h   # a carry rolls into the exponent
    return sign or uint16(h)
  if a < 0x33000000'u32: return sign                          # below 2^-25: rounds to zero
  # subnormal half: units of 2^-24.  |f| = m * 2^(e - 150) with the 24-bit significand m, so the result is m >> (126 - e)
  let e = a shr 23
  let m = (a and 0x7FFFFF'u32) or 0x800000'u32
  let shift = 126'u32 - e                                     # 14 .. 24
  var r = m shr shift
  let rem = m and ((1'u32 shl shift) - 1'u32)
  let halfway = 1'u32 shl (shift - 1'u32)
  if rem > halfway or (rem == halfway and (r and 1'u32) == 1'u32): inc r
  return sign or uint16(r)

proc halfRows(m: var Model, names: openArray[string]): seq[uint16] =
  ## The named float32 tensors, one after the other, as fp16 bit patterns, rounded to nearest even.  F16 GGUF
  ## values convert exactly.
  for name in names:
    let t = m.getTensor(name)
    let base = result.len
    result.setLen(base + t.data.len)
    for i, v in t.data:
      result[base + i] = floatToHalfRne(v)

proc floatRows(m: var Model, names: openArray[string]): seq[float32] =
  for name in names:
    result.add m.getTensor(name).data

proc loadModelBackend*(m: var Model, hp: HParams) =
  when defined(b200Standin):
    ## Stand-in weights: the four tables are read from tensors named like this in `m`.
    var eq = m.getTensor("standin.eq")
    var ek = m.getTensor("standin.ek")
    var ev = m.getTensor("standin.ev")
    var wout = m.getTensor("standin.wout")
    var w = HlStandinWeights(eq: addr eq.data[0], ek: addr ek.data[0], ev: addr ev.data[0],
                             wout: addr wout.data[0], qNorm: nil, kNorm: nil)
    shimHp = toHl(hp)
    check hl_backend_load_model(0, addr shimHp, addr w)
  else:
    ## Dense llama / qwen3: the tensors ensureModelGpuPtrs uploads for lkAttentionFfn layers
    ## (naive.nim:3610-3700, 3811-3846), gathered per kind over all layers.
    if m.infos.hasKey("blk.0.ffn_gate_inp.weight") or m.infos.hasKey("blk.0.ssm_conv1d.weight"):
      raise newException(ValueError, "b200 backend: MoE and SSM layers are not supported (dense llama / qwen3 only)")
    proc names(suffix: string): seq[string] =
      for l in 0 ..< hp.nLayer: result.add "blk." & $l & "." & suffix
    let hasQkNorm = m.infos.hasKey("blk.0.attn_q_norm.weight")
    let outName = if m.infos.hasKey("output.weight"): "output.weight" else: "token_embd.weight"  # tied embeddings
    var
      tokEmb = halfRows(m, ["token_embd.weight"])
      wq = halfRows(m, names("attn_q.weight"))
      wk = halfRows(m, names("attn_k.weight"))
      wv = halfRows(m, names("attn_v.weight"))
      wo = halfRows(m, names("attn_output.weight"))
      wGate = halfRows(m, names("ffn_gate.weight"))
      wUp = halfRows(m, names("ffn_up.weight"))
      wDown = halfRows(m, names("ffn_down.weight"))
      wOut = halfRows(m, [outName])
      attnNorm = floatRows(m, names("attn_norm.weight"))
      ffnNorm = floatRows(m, names("ffn_norm.weight"))
      outNorm = floatRows(m, ["output_norm.weight"])
      qNorm = if hasQkNorm: floatRows(m, names("attn_q_norm.weight")) else: @[]
      kNorm = if hasQkNorm: floatRows(m, names("attn_k_norm.weight")) else: @[]
    var w = HlDenseWeights(
      tokEmb: addr tokEmb[0], attnNorm: addr attnNorm[0], wq: addr wq[0], wk: addr wk[0], wv: addr wv[0],
      wo: addr wo[0], qNorm: (if hasQkNorm: addr qNorm[0] else: nil), kNorm: (if hasQkNorm: addr kNorm[0] else: nil),
      ffnNorm: addr ffnNorm[0], wGate: addr wGate[0], wUp: addr wUp[0], wDown: addr wDown[0],
      outNorm: addr outNorm[0], wOut: addr wOut[0])
    shimDenseHp = toDense(hp)
    check hl_dense_load_model(0, addr shimDenseHp, addr w)   # the library copies everything to the device

proc unloadModelBackend*() =
  for key in toSeq(shimCaches.keys):
    when defined(b200Standin):
      discard hl_backend_free_kv_cache(addr shimCaches[key])
    else:
      discard hl_dense_free_kv_cache(addr shimCaches[key])
  shimCaches.clear()
  when defined(b200Standin):
    check hl_backend_unload_model()
  else:
    check hl_dense_unload_model()

proc forwardPrefill*(m: var Model, tokens: seq[int32], cache: var KvCache): Tensor =
  if tokens.len == 0:
    raise newException(ValueError, "prefill requires at least one token")
  result = newTensor(@[1, m.hparams.nVocab])      # last position only, like megakernel.nim:2498
  let shim = syncIn(cache)
  when defined(b200Standin):
    check hl_backend_forward_prefill(unsafeAddr tokens[0], tokens.len.int32, shim, addr result.data[0])
  else:
    check hl_dense_forward_prefill(unsafeAddr tokens[0], tokens.len.int32, shim, addr result.data[0])
  syncOut(cache, shim)

proc forwardDecode*(m: var Model, token: int32, cache: var KvCache): Tensor =
  result = newTensor(@[1, m.hparams.nVocab])
  let shim = syncIn(cache)
  when defined(b200Standin):
    check hl_backend_forward_decode(token, shim, addr result.data[0])
  else:
    check hl_dense_forward_decode(token, shim, addr result.data[0])
  syncOut(cache, shim)

proc forwardDecodeToken*(m: var Model, token: int32, cache: var KvCache): int32 =
  let shim = syncIn(cache)
  when defined(b200Standin):
    check hl_backend_forward_decode_token(token, shim, addr result)
  else:
    check hl_dense_forward_decode_token_timed(token, shim, addr result, nil)
  syncOut(cache, shim)

proc forwardDecodeTokenTimed*(m: var Model, token: int32, cache: var KvCache,
                              gpuMs: var float32): int32 =
  let shim = syncIn(cache)
  when defined(b200Standin):
    check hl_backend_forward_decode_token_timed(token, shim, addr result, addr gpuMs)
  else:
    check hl_dense_forward_decode_token_timed(token, shim, addr result, addr gpuMs)
  syncOut(cache, shim)
