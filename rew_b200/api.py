"""Host-side mirror of the rew interfaces this backend stands behind.

Names and argument meaning follow rew (Nim): Tensor/fromHost/toHost
(src/rew/eager.nim:360-377,558-595), Linear (src/rew/nn/linear.nim), rmsNorm and
LayerNorm (src/rew/nn/norm.nim), RotaryPositionEncoding (src/rew/nn/rope.nim),
scaledDotProductAttention (src/rew/nn/attention.nim), GatedFeedForward
(src/rew/nn/gated_ffn.nim), Embedding (src/rew/nn/embedding.nim), the causal-LM
models (src/rew/models/llama.nim, deepseek.nim) and generate
(src/rew/infer/generate.nim).  Everything here is a thin ctypes call into
librew_b200.so; there is no Python or CPU implementation of any op.
"""
import ctypes as C
import weakref

import numpy as np

from . import _lib
from ._lib import BF16, F32, I32, RewB200Error, check, lib
from .weights import ModelConfig, from_bf16_bits, tensor_specs, to_bf16_bits

_NP = {F32: np.float32, I32: np.int32, _lib.I64: np.int64, _lib.F64: np.float64, _lib.U8: np.uint8,
       _lib.BOOL: np.bool_, _lib.I8: np.int8, _lib.I16: np.int16}


class Tensor:
    """Owning handle of one device buffer (rew's BufferHandle + Tensor metadata)."""

    def __init__(self, handle):
        self._h = C.c_void_p(handle) if not isinstance(handle, C.c_void_p) else handle
        dt = C.c_int32()
        nd = C.c_int32()
        dims = (C.c_int64 * 8)()
        check(lib().rewb200_buffer_info(self._h, C.byref(dt), dims, C.byref(nd)))
        self.dtype = dt.value
        self.shape = tuple(dims[i] for i in range(nd.value))

    @staticmethod
    def from_host(array, dtype=None, slot=0):
        """fromHost: uploads a numpy array.  dtype=BF16 rounds f32 data to bf16 (RNE)."""
        _lib.init()
        a = np.ascontiguousarray(array)
        if dtype is None:
            dtype = {np.dtype(np.float32): F32, np.dtype(np.int32): I32, np.dtype(np.int64): _lib.I64,
                     np.dtype(np.float64): _lib.F64}[a.dtype]
        if dtype == BF16:
            payload = to_bf16_bits(a.astype(np.float32))
        else:
            payload = np.ascontiguousarray(a.astype(_NP[dtype]))
        dims = (C.c_int64 * max(1, a.ndim))(*a.shape)
        out = C.c_void_p()
        check(lib().rewb200_buffer_from_host(slot, payload.ctypes.data_as(C.c_void_p), dtype, dims, a.ndim, C.byref(out)))
        return Tensor(out)

    def to_host(self):
        """toHost: bf16 buffers come back widened to float32."""
        n = int(np.prod(self.shape)) if self.shape else 1
        if self.dtype == BF16:
            raw = np.empty(n, np.uint16)
            check(lib().rewb200_buffer_to_host(self._h, raw.ctypes.data_as(C.c_void_p), raw.nbytes))
            return from_bf16_bits(raw).reshape(self.shape)
        raw = np.empty(n, _NP[self.dtype])
        check(lib().rewb200_buffer_to_host(self._h, raw.ctypes.data_as(C.c_void_p), raw.nbytes))
        return raw.reshape(self.shape)

    def release(self):
        if self._h is not None and self._h.value:
            lib().rewb200_buffer_release(self._h)
        self._h = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def _out():
    return C.c_void_p()


def _h(t):
    return t._h if t is not None else None


class Linear:
    """y = x @ weight + bias, weight [in,out] (src/rew/nn/linear.nim:21-49)."""

    def __init__(self, weight, bias):
        self.weight, self.bias = weight, bias

    def forward(self, x):
        o = _out()
        check(lib().rewb200_linear(_h(x), _h(self.weight), _h(self.bias), C.byref(o)))
        return Tensor(o)


class QloraLinear:
    """QloraLinear (src/rew/nn/lora.nim:173-191,331-431) with the frozen weight kept as NF4 codes on the
    device.  weight: Tensor [in,out] f32 or bf16 (quantised here, blocks of 64); bias f32 [out] or None;
    A f32 [rank,in], B f32 [out,rank] or None; scaling = alpha / rank."""

    def __init__(self, weight, bias=None, A=None, B=None, scaling=1.0):
        h = C.c_void_p()
        check(lib().rewb200_nf4_pack(_h(weight), C.byref(h)))
        self._q, self.bias, self.A, self.B, self.scaling = h, bias, A, B, float(scaling)
        k, n = C.c_int64(), C.c_int64()
        check(lib().rewb200_nf4_info(self._q, C.byref(k), C.byref(n)))
        self.inFeatures, self.outFeatures = k.value, n.value

    def forward(self, x):
        o = _out()
        check(lib().rewb200_qlora_linear(_h(x), self._q, _h(self.bias), _h(self.A), _h(self.B), self.scaling, C.byref(o)))
        return Tensor(o)

    def unpack(self):
        """(packed uint8 [in*out/2], scales f32 [in*out/64]) in the reference's nf4Quantize format."""
        n = self.inFeatures * self.outFeatures
        packed, scales = np.empty(n // 2, np.uint8), np.empty(n // 64, np.float32)
        check(lib().rewb200_nf4_unpack(self._q, packed.ctypes.data_as(C.POINTER(C.c_uint8)), scales.ctypes.data_as(_lib.F32P)))
        return packed, scales

    def dequantized_weight(self):
        o = _out()
        check(lib().rewb200_nf4_dequantize(self._q, C.byref(o)))
        return Tensor(o)

    def release(self):
        if self._q is not None:
            lib().rewb200_nf4_free(self._q)
            self._q = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def rmsNorm(x, gamma, eps=1e-5):
    o = _out()
    check(lib().rewb200_rmsnorm(_h(x), _h(gamma), eps, C.byref(o)))
    return Tensor(o)


class LayerNorm:
    def __init__(self, gamma, beta, eps=1e-5):
        self.gamma, self.beta, self.eps = gamma, beta, eps

    def forward(self, x):
        o = _out()
        check(lib().rewb200_layernorm(_h(x), _h(self.gamma), _h(self.beta), self.eps, C.byref(o)))
        return Tensor(o)


class RotaryPositionEncoding:
    """initRotaryPositionEncoding + forward (src/rew/nn/rope.nim:112-179)."""

    def __init__(self, headDim, maxSeqLen=2048, theta=10000.0, slot=0):
        _lib.init()
        c, s = _out(), _out()
        check(lib().rewb200_rope_tables(slot, headDim, maxSeqLen, float(theta), C.byref(c), C.byref(s)))
        self.cosCached, self.sinCached = Tensor(c), Tensor(s)
        self.headDim, self.maxSeqLen, self.theta = headDim, maxSeqLen, theta

    def forward(self, x, offset=0):
        o = _out()
        check(lib().rewb200_rope(_h(x), _h(self.cosCached), _h(self.sinCached), offset, C.byref(o)))
        return Tensor(o)


def scaledDotProductAttention(q, k, v, causal=False, mask_kind=0):
    """q [B,nh,S,hd]; k, v [B,kvh,L,hd] (kv heads are shared by nh/kvh query heads)."""
    o = _out()
    check(lib().rewb200_gqa_attention(_h(q), _h(k), _h(v), int(bool(causal)), mask_kind, C.byref(o)))
    return Tensor(o)


class GatedFeedForward:
    def __init__(self, gateProj, upProj, downProj):
        self.gateProj, self.upProj, self.downProj = gateProj, upProj, downProj

    def forward(self, x):
        o = _out()
        check(lib().rewb200_swiglu_ffn(_h(x), _h(self.gateProj.weight), _h(self.gateProj.bias), _h(self.upProj.weight),
                                       _h(self.upProj.bias), _h(self.downProj.weight), _h(self.downProj.bias), C.byref(o)))
        return Tensor(o)


class Embedding:
    def __init__(self, weight):
        self.weight = weight

    def forward(self, ids):
        o = _out()
        check(lib().rewb200_embed_gather(_h(ids), _h(self.weight), C.byref(o)))
        return Tensor(o)


def moeRoute(x, router, top_k):
    w, i = _out(), _out()
    check(lib().rewb200_moe_route(_h(x), _h(router.weight), _h(router.bias), top_k, C.byref(w), C.byref(i)))
    return Tensor(w), Tensor(i)


class KvCache:
    """KvCache (src/rew/nn/kv_cache.nim:13-24): K and V of one attention layer on the device, appended in place."""

    def __init__(self, batch, numKvHeads, headDim, maxLen, dtype=F32, slot=0):
        _lib.init()
        h = C.c_void_p()
        check(lib().rewb200_kv_create(slot, dtype, batch, numKvHeads, headDim, maxLen, C.byref(h)))
        self._h = h

    @property
    def length(self):
        return lib().rewb200_kv_length(self._h)

    def reset(self):
        check(lib().rewb200_kv_reset(self._h))

    def free(self):
        if self._h is not None:
            lib().rewb200_kv_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class GroupedQueryAttention:
    """GroupedQueryAttention with a cache (src/rew/nn/groupedqueryattention.nim:27-38,94-144): q/k/v Linear,
    RoPE at the cache length, in-place append, attention over the cache, outProj.  x [batch, S, embedDim]."""

    def __init__(self, qProj, kProj, vProj, outProj, rope, mask_kind=0):
        self.qProj, self.kProj, self.vProj, self.outProj, self.rope, self.mask_kind = qProj, kProj, vProj, outProj, rope, mask_kind

    def forward(self, x, cache, causal=True):
        q = _out()
        check(lib().rewb200_qkv_rope_kvappend(_h(x), _h(self.qProj.weight), _h(self.qProj.bias), _h(self.kProj.weight),
                                              _h(self.kProj.bias), _h(self.vProj.weight), _h(self.vProj.bias),
                                              _h(self.rope.cosCached), _h(self.rope.sinCached), cache._h, C.byref(q)))
        q = Tensor(q)
        a = _out()
        check(lib().rewb200_gqa_attention_cached(_h(q), cache._h, int(bool(causal)), self.mask_kind, C.byref(a)))
        a = Tensor(a)
        B, S, nq = a.shape
        flat = reshape(a, (B * S, nq))
        y = self.outProj.forward(flat)
        return reshape(y, (B, S, y.shape[1]))


def reshape(t, shape):
    return dispatch("reshape", [t], [("shape", "[" + ",".join(str(int(v)) for v in shape) + "]")])[0]


class RoutedExperts:
    """The routed experts of a DeepSeekMoE layer (src/rew/models/deepseek.nim:36-52).  experts: a list of
    (gateProj, upProj, downProj) Linear triples; forward applies DeepSeekMoE.forward's weighted sum for the
    routing that moeRoute returned."""

    def __init__(self, experts, slot=0):
        _lib.init()
        n = len(experts)

        def arr(get):
            return (C.c_void_p * n)(*[(_h(get(e)).value if get(e) is not None else None) for e in experts])

        h = C.c_void_p()
        check(lib().rewb200_experts_create(slot, n, arr(lambda e: e[0].weight), arr(lambda e: e[0].bias),
                                           arr(lambda e: e[1].weight), arr(lambda e: e[1].bias),
                                           arr(lambda e: e[2].weight), arr(lambda e: e[2].bias), C.byref(h)))
        self._h = h

    def forward(self, x, weights, indices):
        o = _out()
        check(lib().rewb200_moe_experts(self._h, _h(x), _h(weights), _h(indices), C.byref(o)))
        return Tensor(o)

    def free(self):
        if self._h is not None:
            lib().rewb200_experts_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Sampler:
    """GenerationConfig + Key of generate (src/rew/infer/generate.nim:12-58,231-265) for a batch of sequences."""

    def __init__(self, batch, vocab, max_tokens, temperature=1.0, top_k=50, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
                 do_sample=True, seeds=None, slot=0):
        _lib.init()
        sp = None
        if seeds is not None:
            sd = np.ascontiguousarray(seeds, dtype=np.uint64)
            assert sd.shape == (batch,), "seeds must hold one value per sequence"
            sp = sd.ctypes.data_as(C.POINTER(C.c_uint64))
        h = C.c_void_p()
        check(lib().rewb200_sampler_create(slot, batch, vocab, max_tokens, temperature, top_k, top_p, min_p, repetition_penalty,
                                           int(bool(do_sample)), sp, C.byref(h)))
        self._h, self.batch, self.vocab = h, batch, vocab

    def observe(self, ids):
        a = np.ascontiguousarray(ids, dtype=np.int32).reshape(self.batch, -1)
        check(lib().rewb200_sampler_observe(self._h, a.ctypes.data_as(_lib.I32P), a.shape[1]))

    def free(self):
        if self._h is not None:
            lib().rewb200_sampler_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def lmHeadSample(x, lmHead, sampler=None, want_logits=False):
    """lmHead + sampleGreedy / sampleTopK / sampleTopP on the last hidden state x [batch, d]; returns ids (and logits)."""
    B, V = x.shape[0], lmHead.weight.shape[1]
    ids = np.empty(B, np.int32)
    logits = np.empty((B, V), np.float32) if want_logits else None
    check(lib().rewb200_lmhead_sample(_h(x), _h(lmHead.weight), _h(lmHead.bias), sampler._h if sampler is not None else None,
                                      ids.ctypes.data_as(_lib.I32P), logits.ctypes.data_as(_lib.F32P) if want_logits else None))
    return (ids, logits) if want_logits else ids


def dispatch(op, operands, attrs=()):
    """dispatchEager(op, operands, attrs) (src/rew/dispatch.nim:75-85)."""
    n = len(operands)
    arr = (C.c_void_p * max(1, n))(*[t._h for t in operands])
    keys = (C.c_char_p * max(1, len(attrs)))(*[k.encode() for k, _ in attrs])
    vals = (C.c_char_p * max(1, len(attrs)))(*[v.encode() for _, v in attrs])
    outs = (C.c_void_p * 4)()
    n_out = C.c_int32(4)
    check(lib().rewb200_dispatch(op.encode(), arr, n, keys, vals, len(attrs), outs, C.byref(n_out)))
    return [Tensor(C.c_void_p(outs[i])) for i in range(n_out.value)]


class CausalLM:
    """LlamaForCausalLM / DeepSeekForCausalLM on the device."""

    def __init__(self, cfg: ModelConfig, slot=0):
        _lib.init()
        self.cfg = cfg
        self._c = cfg.to_c()
        h = C.c_void_p()
        check(lib().rewb200_model_create(slot, C.byref(self._c), C.byref(h)))
        self._h = h
        self._sessions = weakref.WeakSet()  # sessions point into the model: they are freed first

    def load(self, tensors):
        """tensors: float32 arrays in canonical order (weights.tensor_specs)."""
        specs = tensor_specs(self.cfg)
        assert len(tensors) == len(specs) == lib().rewb200_model_tensor_count(self._h)
        for i, (t, (name, shape)) in enumerate(zip(tensors, specs)):
            a = np.ascontiguousarray(t, dtype=np.float32)
            assert a.shape == tuple(shape), (name, a.shape, shape)
            check(lib().rewb200_model_set_tensor(self._h, i, a.ctypes.data_as(_lib.F32P), a.size))
        check(lib().rewb200_model_finalize(self._h))
        return self

    def tensor_layout(self, index):
        """(global_shape, local_shape, offsets, partitioned_dim) of logical tensor `index` on this rank: shardLayout's
        block rule (src/rew/sharding.nim:255-270) for the model's tensor- / expert-parallel placement."""
        nd, pd = C.c_int32(), C.c_int32()
        g, l, o = (C.c_int64 * 4)(), (C.c_int64 * 4)(), (C.c_int64 * 4)()
        check(lib().rewb200_model_tensor_layout(self._h, index, C.byref(nd), g, l, o, C.byref(pd)))
        n = nd.value
        return tuple(g[:n]), tuple(l[:n]), tuple(o[:n]), pd.value

    def load_shards(self, get_block):
        """Uploads only this rank's block of every tensor.  get_block(index, name, global_shape, local_shape,
        offsets) returns that block as a float32 array of local_shape (it is not called for tensors another
        rank owns)."""
        specs = tensor_specs(self.cfg)
        assert len(specs) == lib().rewb200_model_tensor_count(self._h)
        for i, (name, shape) in enumerate(specs):
            g, l, o, _ = self.tensor_layout(i)
            assert tuple(g) == tuple(shape), (name, g, shape)
            if 0 in l:
                continue
            a = np.ascontiguousarray(get_block(i, name, g, l, o), dtype=np.float32)
            assert a.shape == tuple(l), (name, a.shape, l)
            nd = len(l)
            check(lib().rewb200_model_set_tensor_shard(self._h, i, a.ctypes.data_as(_lib.F32P), (C.c_int64 * nd)(*l),
                                                       (C.c_int64 * nd)(*o), nd))
        check(lib().rewb200_model_finalize(self._h))
        return self

    def load_checkpoint(self, path):
        """A rew checkpoint directory straight into this rank's buffers: of a sharded leaf only the shard files
        that overlap this rank's block are read (rew_b200.checkpoint.read_block)."""
        from . import checkpoint as CK
        reader = CK.BlockReader(path, self.cfg)
        return self.load_shards(lambda i, name, g, l, o: reader.read_block(name, l, o))

    @classmethod
    def from_hf_snapshot(cls, snap_dir, dtype=None, slot=0, **config_overrides):
        """A Hugging Face Llama snapshot directory (config.json + one or more *.safetensors) on the device:
        hfDownloadModel's layout read the way loadHfConfig / toLlamaConfig / loadSafetensorsWeights do
        (src/rew/hf/hub.nim:344-394), with the tensor mapping that loadLlamaWeights leaves out."""
        import os
        from . import safetensors as st
        cfg = st.llama_config_from_hf(os.path.join(snap_dir, "config.json"), dtype=dtype, **config_overrides)
        return cls(cfg, slot).load(st.llama_from_hf(cfg, st.read_safetensors_dir(snap_dir)))

    def init_random(self, seed=0, std=0.02):
        check(lib().rewb200_model_init_random(self._h, seed, std))
        check(lib().rewb200_model_finalize(self._h))
        return self

    def weight_bytes(self):
        return lib().rewb200_model_weight_bytes(self._h)

    def session(self, batch, max_len):
        s = Session(self, batch, max_len)
        self._sessions.add(s)
        return s

    def paged_session(self, lanes, max_len, num_blocks):
        s = PagedSession(self, lanes, max_len, num_blocks)
        self._sessions.add(s)
        return s

    def free(self):
        if self._h is not None:
            for s in list(self._sessions):
                s.free()
            lib().rewb200_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Session:
    """A batch of sequences with its paged KV cache."""

    def __init__(self, model, batch, max_len):
        self.model, self.batch, self.max_len = model, batch, max_len
        h = C.c_void_p()
        check(lib().rewb200_session_create(model._h, batch, max_len, C.byref(h)))
        self._h = h

    def _ids(self, ids):
        a = np.ascontiguousarray(ids, dtype=np.int32)
        if a.ndim == 1:
            a = a.reshape(1, -1)
        assert a.shape[0] == self.batch, "ids must be [batch, S]"
        return a

    def forward(self, ids, want_logits=False):
        a = self._ids(ids)
        nxt = np.empty(self.batch, np.int32)
        logits = np.empty((self.batch, self.model.cfg.vocab), np.float32) if want_logits else None
        check(lib().rewb200_session_forward(self._h, a.ctypes.data_as(_lib.I32P), a.shape[1], nxt.ctypes.data_as(_lib.I32P),
                                            logits.ctypes.data_as(_lib.F32P) if want_logits else None))
        return (nxt, logits) if want_logits else nxt

    def decode(self, n_steps, want_logits=False):
        out = np.empty((self.batch, n_steps), np.int32)
        logits = np.empty((self.batch, self.model.cfg.vocab), np.float32) if want_logits else None
        check(lib().rewb200_session_decode(self._h, n_steps, out.ctypes.data_as(_lib.I32P),
                                           logits.ctypes.data_as(_lib.F32P) if want_logits else None))
        return (out, logits) if want_logits else out

    def generate(self, prompt, max_new_tokens, eos=-1, want_logits=False, stop_ids=()):
        """generate (src/rew/infer/generate.nim:231-265), batched; stop_ids = GenerationConfig.stopTokenIds."""
        a = self._ids(prompt)
        out = np.empty((self.batch, max_new_tokens), np.int32)
        logits = np.empty((self.batch, self.model.cfg.vocab), np.float32) if want_logits else None
        stops = np.ascontiguousarray(list(stop_ids), dtype=np.int32)
        check(lib().rewb200_generate_stop(self._h, a.ctypes.data_as(_lib.I32P), a.shape[1], max_new_tokens, eos,
                                          stops.ctypes.data_as(_lib.I32P) if stops.size else None, int(stops.size),
                                          out.ctypes.data_as(_lib.I32P), logits.ctypes.data_as(_lib.F32P) if want_logits else None))
        return (out, logits) if want_logits else out

    def routing(self, moe_layer, rows):
        """Expert ids [rows, top_k] MoE layer `moe_layer` chose in the last forward (needs option record_routing=1)."""
        out = np.empty((rows, self.model.cfg.top_k), np.int32)
        check(lib().rewb200_session_routing(self._h, moe_layer, out.ctypes.data_as(_lib.I32P), rows))
        return out

    TRACE_CATEGORIES = ("embed_norm", "qkv_linear", "qkv_post", "attention", "o_linear", "norm_after_attention",
                        "gate_up_linear", "down_linear", "routed_experts", "norm_after_ffn", "head_and_next_token")

    def trace_step(self):
        """One decode step with a CUDA event after every category of launches: {category: ms summed over layers}."""
        ms = (C.c_float * 16)()
        check(lib().rewb200_session_trace_step(self._h, ms, 16))
        return {k: float(ms[i]) for i, k in enumerate(self.TRACE_CATEGORIES)}

    def set_sampling(self, temperature=1.0, top_k=50, top_p=1.0, min_p=0.0, repetition_penalty=1.0, do_sample=True,
                     seeds=None):
        """initGenerationConfig (src/rew/infer/generate.nim:30-58) for this session; the defaults are the
        reference's.  seeds: one uint64 per sequence (initKey); None = 0, the reference's default key."""
        sp = None
        if seeds is not None:
            sd = np.ascontiguousarray(seeds, dtype=np.uint64)
            assert sd.shape == (self.batch,), "seeds must hold one value per sequence"
            sp = sd.ctypes.data_as(C.POINTER(C.c_uint64))
        check(lib().rewb200_session_set_sampling(self._h, float(temperature), int(top_k), float(top_p), float(min_p),
                                                 float(repetition_penalty), int(bool(do_sample)), sp))

    def clear_sampling(self):
        check(lib().rewb200_session_clear_sampling(self._h))

    def logprobs(self, n):
        """GenerationResult.logProbs of the first n tokens sampled since the last reset, [batch, n]."""
        out = np.empty((self.batch, n), np.float32)
        check(lib().rewb200_session_logprobs(self._h, n, out.ctypes.data_as(_lib.F32P)))
        return out

    def forward_all(self, ids, offset=0, causal=True):
        """Model.forward without a cache: logits for every position [batch,S,vocab]."""
        a = self._ids(ids)
        logits = np.empty((self.batch, a.shape[1], self.model.cfg.vocab), np.float32)
        check(lib().rewb200_model_forward_all(self._h, a.ctypes.data_as(_lib.I32P), a.shape[1], offset, int(bool(causal)),
                                              logits.ctypes.data_as(_lib.F32P)))
        return logits

    def reset(self):
        check(lib().rewb200_session_reset(self._h))

    def last_ms(self):
        p, d = C.c_float(), C.c_float()
        check(lib().rewb200_session_last_ms(self._h, C.byref(p), C.byref(d)))
        return p.value, d.value

    def free(self):
        if self._h is not None:
            if self.model._h is not None:  # a freed model has already released its sessions
                lib().rewb200_session_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PagedSession(Session):
    """Continuous batching: `lanes` sequences of independent length over a shared pool of KV blocks
    (PagedKvCache, src/rew/infer/generate.nim:63-88).  set_sampling / logprobs / free as Session."""

    def __init__(self, model, lanes, max_len, num_blocks):
        self.model, self.batch, self.max_len, self.num_blocks = model, lanes, max_len, num_blocks
        h = C.c_void_p()
        check(lib().rewb200_session_create_paged(model._h, lanes, max_len, num_blocks, C.byref(h)))
        self._h = h

    def free_blocks(self):
        return int(lib().rewb200_session_free_blocks(self._h))

    def lane_length(self, lane):
        return int(lib().rewb200_lane_length(self._h, lane))

    def admit(self, lane, ids, seed=0):
        """Prefills one idle lane with the prompt `ids`; returns its first new token."""
        a = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        nxt = C.c_int32(-1)
        check(lib().rewb200_lane_admit(self._h, lane, a.ctypes.data_as(_lib.I32P), a.size, C.c_uint64(seed), C.byref(nxt)))
        return int(nxt.value)

    def step(self, n_steps=1):
        """n decode steps for every active lane: ids [lanes, n_steps], -1 for idle lanes."""
        out = np.empty((self.batch, n_steps), np.int32)
        check(lib().rewb200_lanes_step(self._h, n_steps, out.ctypes.data_as(_lib.I32P)))
        return out

    def release(self, lane):
        check(lib().rewb200_lane_release(self._h, lane))


def set_option(key, value, slot=0):
    """rewb200_set_option: run-time switches such as ("linear", "tc")."""
    _lib.init()
    check(lib().rewb200_set_option(slot, key.encode(), value.encode()))


def comm_unique_id():
    """128-byte NCCL id, created on rank 0 and handed to every rank by the host program."""
    buf = C.create_string_buffer(128)
    check(lib().rewb200_comm_unique_id(buf))
    return buf.raw


def comm_init(unique_id, rank, world, slot=0):
    _lib.init()
    check(lib().rewb200_comm_init(slot, C.create_string_buffer(unique_id, 128), rank, world))


def comm_destroy(slot=0):
    check(lib().rewb200_comm_destroy(slot))


def comm_peer_alloc(allreduce_bytes, alltoall_bytes=0, slot=0):
    """Allocates this rank's peer heap (fused all-reduce slots and the expert-parallel all-to-all region);
    returns its 64-byte IPC handle."""
    buf = C.create_string_buffer(64)
    check(lib().rewb200_comm_peer_alloc(slot, int(allreduce_bytes), int(alltoall_bytes), buf))
    return buf.raw


def comm_peer_attach(handles, slot=0):
    """handles: the 64-byte handles of all ranks, in rank order."""
    blob = b"".join(handles)
    check(lib().rewb200_comm_peer_attach(slot, C.create_string_buffer(blob, len(blob))))
