## Eager backend for rew that calls librew_b200.so (B200, sm_100a).
##
## A rew maintainer drops this file and rew_b200_abi.nim (generated from include/rew_b200.h by
## nim/gen_importc.py) into src/rew/backends/ and calls `installB200Backend()` instead of
## `installEagerBackend()` (src/rew/eager.nim:1769-1772).  It replaces, for the decoder-inference path:
##   - the EagerBackend proc slot (src/rew/dispatch.nim:47-49,65-68)         -> rewb200_dispatch
##   - transferToDevice / transferToHost (src/rew/eager.nim:229-247)          -> rewb200_buffer_from_host / _to_host
##   - the BufferReleaser of device buffers (src/rew/buffer.nim:33,69-82)     -> rewb200_buffer_release
## and offers the fused forwards further down for backend-aware rew.nn layers.
##
## Written against the reference's signatures:
##   initEagerTensor(buffer: BufferHandle; dtype: DType; shape: openArray[int]; device: Device;
##                   sharding = initReplicated())                              src/rew/tensor.nim:130-133
##   newBufferHandle(target, raw: PjrtBufferRaw, releaser, sizeBytes = 0)      src/rew/buffer.nim:85-96
##   EagerError = object of CatchableError                                     src/rew/eager.nim:42-45
##   parseDevice("target[:ordinal]")                                           src/rew/device.nim:66-98
## There is no Nim toolchain where this library is built, so this file is checked only by
## tests/test_host.py (every C name used here exists in the header) and by reading.
import std/[strutils, sequtils]
import ../tensor, ../buffer, ../dtype, ../device, ../dispatch, ../sharding
from ../eager import EagerError
import ./rew_b200_abi

proc check(st: cint) =
  ## Status codes never escape into rew: they become EagerError with the library's message.
  if st != REWB200_OK:
    raise newException(EagerError, $rewb200_last_error())

proc b200Releaser(target: Target; raw: PjrtBufferRaw) {.nimcall, raises: [].} =
  ## nil-safe and callable from whichever thread drops the last reference; each raw is wrapped exactly once.
  rewb200_buffer_release(cast[ptr RewbBuffer](raw))

proc rawOf(t: Tensor): ptr RewbBuffer =
  if t.buffer.isNil:
    raise newException(TensorError, "b200 backend: tensor has no device buffer (trace tensor in eager mode?)")
  cast[ptr RewbBuffer](t.buffer.raw)

proc wrap(raw: ptr RewbBuffer; device: Device; sharding: Sharding): Tensor =
  ## Fresh BufferHandle (ARC) around a buffer the library returned; DType ordinals are shared with the header.
  var dt, nd: cint
  var dims: array[8, int64]
  check rewb200_buffer_info(raw, addr dt, addr dims[0], addr nd)
  var shape = newSeq[int](nd)
  var count = 1
  for i in 0 ..< int(nd):
    shape[i] = int(dims[i])
    count *= shape[i]
  let h = newBufferHandle(device.target, cast[PjrtBufferRaw](raw), b200Releaser,
                          sizeBytes = count * dtypeSizeBytes(DType(dt)))
  initEagerTensor(h, DType(dt), shape, device, sharding)

proc b200Backend(op: string; operands: openArray[Tensor];
    attrs: openArray[(string, string)]): seq[Tensor] {.nimcall, raises: [CatchableError].} =
  ## dispatchEager's target.  Operands must live on one device (src/rew/eager.nim:1726-1729); a zero-operand
  ## op (iota) names its device in the "device" attribute (src/rew/ops/shape.nim:295-323); the result inherits
  ## operands[0].sharding when there is an operand (src/rew/eager.nim:1764-1767).
  var device = defaultDevice()
  var sharding = initReplicated()
  if operands.len > 0:
    device = operands[0].device
    sharding = operands[0].sharding
    for t in operands:
      if t.device != device:
        raise newException(DeviceError, "cross-device operands forbidden: " & $device & " vs " & $t.device)
  else:
    for (k, v) in attrs:
      if k == "device": device = parseDevice(v)
  var raws = newSeq[ptr RewbBuffer](operands.len)
  for i, t in operands: raws[i] = rawOf(t)
  let keys = attrs.mapIt(it[0])
  let vals = attrs.mapIt(it[1])
  let ck = allocCStringArray(keys)
  let cv = allocCStringArray(vals)
  defer:
    deallocCStringArray(ck)
    deallocCStringArray(cv)
  var outs: array[4, ptr RewbBuffer]
  var nOut = cint(4)
  check rewb200_dispatch(op.cstring, (if raws.len > 0: addr raws[0] else: nil), cint(raws.len), ck, cv,
                         cint(attrs.len), addr outs[0], addr nOut)
  for i in 0 ..< int(nOut): result.add wrap(outs[i], device, sharding)

proc b200TransferToDevice*(d: Device; data: pointer; dt: DType; dims: openArray[int]): Tensor =
  ## transferToDevice / fromHost (src/rew/eager.nim:229-235,360-377).
  var d64 = dims.mapIt(int64(it))
  var raw: ptr RewbBuffer
  check rewb200_buffer_from_host(cint(d.ordinal), data, cint(ord(dt)), (if d64.len > 0: addr d64[0] else: nil),
                                 cint(d64.len), addr raw)
  wrap(raw, d, initReplicated())

proc b200TransferToHost*(t: Tensor; dst: pointer; dstSize: int) =
  ## transferToHost / toHost (src/rew/eager.nim:237-247,558-595): synchronous on observation.
  check rewb200_buffer_to_host(rawOf(t), dst, csize_t(dstSize))

proc installB200Backend*(ordinals: openArray[int] = [0]) =
  ## Slot i of the library drives CUDA device ordinals[i]; Device.ordinal indexes slots.
  var o = ordinals.mapIt(cint(it))
  check rewb200_init(addr o[0], cint(o.len))
  setEagerBackend(b200Backend)          # src/rew/dispatch.nim:65-68 (per-thread slot)

# ---- fused forwards (Tier B): same Nim signatures as the rew.nn procs they stand behind ---------------

proc one(call: proc (o: ptr ptr RewbBuffer): cint; like: Tensor): Tensor =
  var raw: ptr RewbBuffer
  check call(addr raw)
  wrap(raw, like.device, like.sharding)

proc linearB200*(x, weight, bias: Tensor): Tensor =
  ## Linear.forward (src/rew/nn/linear.nim:43-49)
  one(proc (o: ptr ptr RewbBuffer): cint = rewb200_linear(rawOf(x), rawOf(weight), rawOf(bias), o), x)

proc rmsNormB200*(x, gamma: Tensor; eps = 1e-5'f32): Tensor =
  ## rmsNorm (src/rew/nn/norm.nim:204-224)
  one(proc (o: ptr ptr RewbBuffer): cint = rewb200_rmsnorm(rawOf(x), rawOf(gamma), cfloat(eps), o), x)

proc layerNormB200*(x, gamma, beta: Tensor; eps = 1e-5'f32): Tensor =
  ## LayerNorm.forward (src/rew/nn/norm.nim:41-84)
  one(proc (o: ptr ptr RewbBuffer): cint = rewb200_layernorm(rawOf(x), rawOf(gamma), rawOf(beta), cfloat(eps), o), x)

proc gatedFfnB200*(x, gateW, gateB, upW, upB, downW, downB: Tensor): Tensor =
  ## GatedFeedForward.forward (src/rew/nn/gated_ffn.nim:46-67)
  one(proc (o: ptr ptr RewbBuffer): cint =
        rewb200_swiglu_ffn(rawOf(x), rawOf(gateW), rawOf(gateB), rawOf(upW), rawOf(upB), rawOf(downW), rawOf(downB), o), x)

proc embeddingB200*(ids, table: Tensor): Tensor =
  ## Embedding.forward on token ids instead of one-hot rows (src/rew/nn/embedding.nim:39-62)
  one(proc (o: ptr ptr RewbBuffer): cint = rewb200_embed_gather(rawOf(ids), rawOf(table), o), table)

type
  KvCacheB200* = object
    ## KvCache (src/rew/nn/kv_cache.nim:13-24) appended in place on the device
    h: ptr RewbKv

proc `=destroy`*(c: KvCacheB200) {.raises: [].} =
  if c.h != nil: rewb200_kv_free(c.h)

proc initKvCacheB200*(d: Device; dt: DType; batch, numKvHeads, headDim, maxLen: int): KvCacheB200 =
  check rewb200_kv_create(cint(d.ordinal), cint(ord(dt)), cint(batch), cint(numKvHeads), cint(headDim), cint(maxLen),
                          addr result.h)

proc length*(c: KvCacheB200): int = int(rewb200_kv_length(c.h))

proc gqaForwardB200*(x, wq, bq, wk, bk, wv, bv, wo, bo, cosT, sinT: Tensor; cache: var KvCacheB200;
                     causal = true; maskKind = 0): Tensor =
  ## GroupedQueryAttention.forward with a cache (src/rew/nn/groupedqueryattention.nim:94-144): x [B, S, d]
  var q, a: ptr RewbBuffer
  check rewb200_qkv_rope_kvappend(rawOf(x), rawOf(wq), rawOf(bq), rawOf(wk), rawOf(bk), rawOf(wv), rawOf(bv),
                                  rawOf(cosT), rawOf(sinT), cache.h, addr q)
  let qT = wrap(q, x.device, x.sharding)
  check rewb200_gqa_attention_cached(rawOf(qT), cache.h, cint(ord(causal)), cint(maskKind), addr a)
  let aT = wrap(a, x.device, x.sharding)
  let rows = aT.shape[0] * aT.shape[1]
  linearB200(aT.reshape([rows, aT.shape[2]]), wo, bo).reshape([aT.shape[0], aT.shape[1], wo.shape[1]])

proc moeRouteB200*(x, routerW, routerB: Tensor; topK: int): tuple[weights, indices: Tensor] =
  ## router of DeepSeekMoE.forward (src/rew/models/deepseek.nim:132-138)
  var w, i: ptr RewbBuffer
  check rewb200_moe_route(rawOf(x), rawOf(routerW), rawOf(routerB), cint(topK), addr w, addr i)
  (wrap(w, x.device, x.sharding), wrap(i, x.device, x.sharding))

proc generateB200*(sess: ptr RewbSession; tokenIds: seq[int32]; maxNewTokens: int; eosTokenId = 2;
                   stopTokenIds: seq[int32] = @[]): seq[int32] =
  ## generate (src/rew/infer/generate.nim:231-265) for a batch-1 session; ids after the first stop token are dropped.
  result = newSeq[int32](maxNewTokens)
  check rewb200_generate_stop(sess, unsafeAddr tokenIds[0], cint(tokenIds.len), cint(maxNewTokens), cint(eosTokenId),
                              (if stopTokenIds.len > 0: unsafeAddr stopTokenIds[0] else: nil), cint(stopTokenIds.len),
                              addr result[0], nil)
  let cut = result.find(-1'i32)
  if cut >= 0: result.setLen(cut)

type
  RoutedExpertsB200* = object
    ## the routed experts of one DeepSeekMoE layer in the backend's fused layout
    ## (src/rew/models/deepseek.nim:74-78,122-145)
    h: ptr RewbExperts

proc `=destroy`*(e: RoutedExpertsB200) {.raises: [].} =
  if e.h != nil: rewb200_experts_free(e.h)

proc initRoutedExpertsB200*(d: Device; gateW, gateB, upW, upB, downW, downB: openArray[Tensor]): RoutedExpertsB200 =
  ## one weight / bias tensor per expert, [in, out] as rew.nn.Linear keeps them
  var gw = gateW.mapIt(rawOf(it))
  var gb = gateB.mapIt(rawOf(it))
  var uw = upW.mapIt(rawOf(it))
  var ub = upB.mapIt(rawOf(it))
  var dw = downW.mapIt(rawOf(it))
  var db = downB.mapIt(rawOf(it))
  check rewb200_experts_create(cint(d.ordinal), cint(gw.len), addr gw[0], addr gb[0], addr uw[0], addr ub[0], addr dw[0],
                               addr db[0], addr result.h)

proc moeExpertsB200*(e: RoutedExpertsB200; x, weights, indices: Tensor): Tensor =
  ## DeepSeekMoE.forward after the router (src/rew/models/deepseek.nim:140-144); weights / indices as moeRouteB200 returns them
  one(proc (o: ptr ptr RewbBuffer): cint = rewb200_moe_experts(e.h, rawOf(x), rawOf(weights), rawOf(indices), o), x)

type
  SamplerB200* = object
    ## GenerationConfig + Key of generate (src/rew/infer/generate.nim:12-58,231-265) held on the device
    h: ptr RewbSampler

proc `=destroy`*(s: SamplerB200) {.raises: [].} =
  if s.h != nil: rewb200_sampler_free(s.h)

proc initSamplerB200*(d: Device; batch, vocab, maxTokens: int; temperature = 1.0'f32; topK = 50; topP = 1.0'f32;
                      minP = 0.0'f32; repetitionPenalty = 1.0'f32; doSample = true; seeds: seq[uint64] = @[]): SamplerB200 =
  check rewb200_sampler_create(cint(d.ordinal), cint(batch), cint(vocab), cint(maxTokens), cfloat(temperature), cint(topK),
                               cfloat(topP), cfloat(minP), cfloat(repetitionPenalty), cint(ord(doSample)),
                               (if seeds.len > 0: unsafeAddr seeds[0] else: nil), addr result.h)

proc observe*(s: SamplerB200; ids: seq[int32]; nPerRow: int) =
  ## the prompt (or any tokens) enters the repetition-penalty history
  check rewb200_sampler_observe(s.h, unsafeAddr ids[0], cint(nPerRow))

proc lmHeadSampleB200*(x, lmW, lmB: Tensor; s: var SamplerB200; batch: int): seq[int32] =
  ## lmHead + lastLogits + sampleGreedy / sampleTopK / sampleTopP (src/rew/infer/generate.nim:92-190) in one call
  result = newSeq[int32](batch)
  check rewb200_lmhead_sample(rawOf(x), rawOf(lmW), rawOf(lmB), s.h, addr result[0], nil)
