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
## Scope: this backend owns the attention path (QK-norm, RoPE, KV append, causal GQA prefill,
## split-KV decode).  The model behind it is the attention-only stand-in of hl_backend.h; a full
## model needs the projection / FFN / vocabulary layers either side of attention, which are not
## part of this library.  No Nim toolchain was available where this file was written: it is a thin
## transliteration of the Python mirror (hippo_leap_b200/backend.py), which IS exercised on a GPU.

when not defined(cpp):
  {.error: "the b200 backend requires Nim's C++ backend. Build with `nim cpp`.".}

import
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
proc hl_b200_kv_layer(kv: pointer, layer: int32, kPool, vPool: ptr pointer,
                      bytesEach: ptr csize_t): int32 {.importc, cdecl, dynlib: hlLib.}

var
  shimCache: HlKvCache          # one model, one cache per process, like naive.nim:235-239
  shimHp: HlHParams

proc check(rc: int32) =
  ## Errors bubble as exceptions (AGENTS.md:224-230); the text comes from the library.
  if rc != 0:
    let msg = $hl_backend_last_error()
    if rc == 4: raise newException(IOError, msg)       # HL_ERR_CUDA
    raise newException(ValueError, msg)

proc toHl(hp: HParams): HlHParams =
  HlHParams(nVocab: hp.nVocab.int32, nLayer: hp.nLayer.int32, nHead: hp.nHead.int32,
            nHeadKv: hp.nHeadKv.int32, headDim: hp.headDim.int32, ropeDim: hp.ropeDim.int32,
            ropeFreqBase: hp.ropeFreqBase, rmsEps: hp.rmsEps,
            ropeMode: HlRopeSplitHalf, llama3Scaling: 0)

proc syncIn(cache: KvCache) =
  ## Callers reset cache.curLen themselves (inference.nim:58); honour it.
  shimCache.curLen = cache.curLen.int32

proc syncOut(cache: var KvCache) =
  cache.curLen = shimCache.curLen.int
  cache.gpuCache.curLen = shimCache.curLen.int     # naive.nim:4586-4587

proc initKvCache*(hp: HParams, maxLen: int): KvCache =
  shimHp = toHl(hp)
  check hl_backend_init_kv_cache(0, addr shimHp, maxLen.int32, addr shimCache)
  result.maxLen = maxLen
  result.curLen = 0
  result.nHeadKv = hp.nHeadKv
  result.headDim = hp.headDim
  result.gpuCache.maxLen = maxLen
  result.gpuCache.nHeadKv = hp.nHeadKv
  result.gpuCache.headDim = hp.headDim
  result.gpuCache.k = newSeq[GpuTensor](hp.nLayer)
  result.gpuCache.v = newSeq[GpuTensor](hp.nLayer)
  let numBlocks = (maxLen + 15) div 16
  for layer in 0 ..< hp.nLayer:
    var kp, vp: pointer
    var bytes: csize_t
    check hl_b200_kv_layer(shimCache.gpuCache, layer.int32, addr kp, addr vp, addr bytes)
    # the layer's page pools: fp16 [numBlocks, nHeadKv, 16, headDim]; `alloc` stays default because
    # the library owns the memory
    result.gpuCache.k[layer] = GpuTensor(devicePtr: kp, shape: @[numBlocks, hp.nHeadKv, 16, hp.headDim],
                                         sizeBytes: bytes.int)
    result.gpuCache.v[layer] = GpuTensor(devicePtr: vp, shape: @[numBlocks, hp.nHeadKv, 16, hp.headDim],
                                         sizeBytes: bytes.int)

proc loadModelBackend*(m: var Model, hp: HParams) =
  ## Stand-in weights: the four tables are read from tensors named like this in `m`.
  var eq = m.getTensor("standin.eq")
  var ek = m.getTensor("standin.ek")
  var ev = m.getTensor("standin.ev")
  var wout = m.getTensor("standin.wout")
  var w = HlStandinWeights(eq: addr eq.data[0], ek: addr ek.data[0], ev: addr ev.data[0],
                           wout: addr wout.data[0], qNorm: nil, kNorm: nil)
  shimHp = toHl(hp)
  check hl_backend_load_model(0, addr shimHp, addr w)

proc unloadModelBackend*() =
  discard hl_backend_free_kv_cache(addr shimCache)
  check hl_backend_unload_model()

proc forwardPrefill*(m: var Model, tokens: seq[int32], cache: var KvCache): Tensor =
  if tokens.len == 0:
    raise newException(ValueError, "prefill requires at least one token")
  result = newTensor(@[1, m.hparams.nVocab])      # last position only, like megakernel.nim:2498
  syncIn(cache)
  check hl_backend_forward_prefill(unsafeAddr tokens[0], tokens.len.int32, addr shimCache,
                                   addr result.data[0])
  syncOut(cache)

proc forwardDecode*(m: var Model, token: int32, cache: var KvCache): Tensor =
  result = newTensor(@[1, m.hparams.nVocab])
  syncIn(cache)
  check hl_backend_forward_decode(token, addr shimCache, addr result.data[0])
  syncOut(cache)

proc forwardDecodeToken*(m: var Model, token: int32, cache: var KvCache): int32 =
  syncIn(cache)
  check hl_backend_forward_decode_token(token, addr shimCache, addr result)
  syncOut(cache)

proc forwardDecodeTokenTimed*(m: var Model, token: int32, cache: var KvCache,
                              gpuMs: var float32): int32 =
  syncIn(cache)
  check hl_backend_forward_decode_token_timed(token, addr shimCache, addr result, addr gpuMs)
  syncOut(cache)
