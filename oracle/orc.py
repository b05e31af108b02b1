"""ctypes binding of the CPU oracle (oracle/rew_oracle.cpp).

Test infrastructure: imported only by tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline legs.  Nothing under rew_b200/ imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liborc.so")


def build(force=False):
    src = os.path.join(HERE, "rew_oracle.cpp")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B", "liborc.so"], check=True, capture_output=True)
    return LIB


class Cfg(C.Structure):
    _fields_ = [
        ("vocab", C.c_int32), ("d_model", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32),
        ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("max_seq", C.c_int32),
        ("theta", C.c_double), ("eps", C.c_float), ("norm_kind", C.c_int32), ("mask_kind", C.c_int32),
        ("n_routed", C.c_int32), ("n_shared", C.c_int32), ("top_k", C.c_int32), ("moe_ffn", C.c_int32),
        ("first_dense", C.c_int32),
    ]


_lib = None
FP = C.POINTER(C.c_float)
IP = C.POINTER(C.c_int32)


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(LIB)
        _lib.orc_reduce_sum.restype = C.c_float
        _lib.orc_log_prob_of.restype = C.c_float
        _lib.orc_tensor_count.restype = C.c_int64
        _lib.orc_decode_bench.restype = C.c_double
    return _lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(FP)


def _ip(a):
    return a.ctypes.data_as(IP)


def cfg_of(mc):
    """ModelConfig-like object (attributes as in rew_b200.weights.ModelConfig) -> Cfg."""
    return Cfg(mc.vocab, mc.d_model, mc.n_layers, mc.n_heads, mc.n_kv_heads, mc.head_dim, mc.ffn, mc.max_seq,
               float(mc.theta), float(mc.eps), mc.norm_kind, mc.mask_kind, mc.n_routed, mc.n_shared, mc.top_k,
               mc.moe_ffn, mc.first_dense)


def _tensor_array(tensors):
    keep = [_f(t) for t in tensors]
    arr = (FP * len(keep))(*[_p(t) for t in keep])
    return keep, arr


def set_accum64(on):
    lib().orc_set_accum64(int(on))


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    """Thread count of the oracle's OpenMP loops; overrides an inherited OMP_NUM_THREADS."""
    lib().orc_set_num_threads(int(n))


def bf16_round(x):
    x = _f(x)
    out = np.empty_like(x)
    lib().orc_bf16_round(_p(x), _p(out), C.c_int64(x.size))
    return out


def binary(op, a, b):
    a, b = _f(a), _f(b)
    out = np.empty_like(a)
    lib().orc_binary({"add": 0, "sub": 1, "mul": 2, "divide": 3}[op], _p(a), _p(b), _p(out), C.c_int64(a.size))
    return out


def unary(op, a):
    a = _f(a)
    out = np.empty_like(a)
    lib().orc_unary({"neg": 0, "exp": 1, "sqrt": 2, "rsqrt": 3, "logistic": 4}[op], _p(a), _p(out), C.c_int64(a.size))
    return out


def matmul(a, b):
    a, b = _f(a), _f(b)
    out = np.empty((a.shape[0], b.shape[1]), np.float32)
    lib().orc_matmul(_p(a), _p(b), _p(out), C.c_int64(a.shape[0]), C.c_int64(a.shape[1]), C.c_int64(b.shape[1]))
    return out


def reduce_sum(a):
    a = _f(a)
    return float(lib().orc_reduce_sum(_p(a), C.c_int64(a.size)))


def transpose2d(a):
    a = _f(a)
    out = np.empty((a.shape[1], a.shape[0]), np.float32)
    lib().orc_transpose2d(_p(a), _p(out), C.c_int64(a.shape[0]), C.c_int64(a.shape[1]))
    return out


def iota2d(rows, cols, dim):
    out = np.empty((rows, cols), np.int32)
    lib().orc_iota2d(_ip(out), C.c_int64(rows), C.c_int64(cols), dim)
    return out


def linear(x, w, b):
    x, w, b = _f(x), _f(w), _f(b)
    y = np.empty((x.shape[0], w.shape[1]), np.float32)
    lib().orc_linear(_p(x), _p(w), _p(b), _p(y), C.c_int64(x.shape[0]), C.c_int64(w.shape[0]), C.c_int64(w.shape[1]))
    return y


def rmsnorm(x, gamma, eps=1e-5):
    x, gamma = _f(x), _f(gamma)
    out = np.empty_like(x)
    d = x.shape[-1]
    lib().orc_rmsnorm(_p(x), _p(gamma), C.c_float(eps), _p(out), C.c_int64(x.size // d), C.c_int64(d))
    return out


def layernorm(x, gamma, beta, eps=1e-5):
    x, gamma, beta = _f(x), _f(gamma), _f(beta)
    out = np.empty_like(x)
    d = x.shape[-1]
    lib().orc_layernorm(_p(x), _p(gamma), _p(beta), C.c_float(eps), _p(out), C.c_int64(x.size // d), C.c_int64(d))
    return out


def rope_tables(hd, max_seq, theta):
    c = np.empty((max_seq, hd), np.float32)
    s = np.empty((max_seq, hd), np.float32)
    lib().orc_rope_tables(hd, max_seq, C.c_double(theta), _p(c), _p(s))
    return c, s


def rope_apply(x, cos_t, sin_t, offset=0):
    x = _f(x)
    out = np.empty_like(x)
    S, hd = x.shape[-2], x.shape[-1]
    lib().orc_rope_apply(_p(x), _p(out), _p(_f(cos_t)), _p(_f(sin_t)), C.c_int64(x.size // (S * hd)), C.c_int64(S), hd,
                         C.c_int64(offset))
    return out


def softmax(x):
    x = _f(x).copy()
    n = x.shape[-1]
    lib().orc_softmax(_p(x), C.c_int64(x.size // n), C.c_int64(n))
    return x


def causal_mask(S, L, mask_kind=0):
    out = np.empty((S, L), np.float32)
    lib().orc_causal_mask(_p(out), C.c_int64(S), C.c_int64(L), mask_kind)
    return out


def gqa_attention(q, k, v, causal=False, mask_kind=0):
    """q [B,nh,S,hd], k,v [B,kvh,L,hd] -> [B,nh,S,hd]."""
    q, k, v = _f(q), _f(k), _f(v)
    B, nh, S, hd = q.shape
    kvh, L = k.shape[1], k.shape[2]
    out = np.empty_like(q)
    lib().orc_gqa_attention(_p(q), _p(k), _p(v), _p(out), C.c_int64(B), nh, kvh, C.c_int64(S), C.c_int64(L), hd,
                            int(bool(causal)), mask_kind)
    return out


def silu(x):
    x = _f(x)
    out = np.empty_like(x)
    lib().orc_silu(_p(x), _p(out), C.c_int64(x.size))
    return out


def gated_ffn(x, gw, gb, uw, ub, dw, db):
    x = _f(x)
    out = np.empty((x.shape[0], dw.shape[1]), np.float32)
    lib().orc_gated_ffn(_p(x), _p(_f(gw)), _p(_f(gb)), _p(_f(uw)), _p(_f(ub)), _p(_f(dw)), _p(_f(db)), _p(out),
                        C.c_int64(x.shape[0]), C.c_int64(x.shape[1]), C.c_int64(gw.shape[1]))
    return out


def embedding_onehot(ids, table):
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    table = _f(table)
    out = np.empty((ids.size, table.shape[1]), np.float32)
    lib().orc_embedding_onehot(_ip(ids), _p(table), _p(out), C.c_int64(ids.size), C.c_int64(table.shape[0]),
                               C.c_int64(table.shape[1]))
    return out.reshape(ids.shape + (table.shape[1],))


def topk(p, k):
    p = _f(p)
    rows, E = p.shape
    vals = np.empty((rows, k), np.float32)
    idx = np.empty((rows, k), np.int32)
    lib().orc_topk(_p(p), C.c_int64(rows), E, k, _p(vals), _ip(idx))
    return vals, idx


def moe_route(x, rw, rb, k):
    x, rw, rb = _f(x), _f(rw), _f(rb)
    N, d = x.shape
    E = rw.shape[1]
    w = np.empty((N, k), np.float32)
    i = np.empty((N, k), np.int32)
    lib().orc_moe_route(_p(x), _p(rw), _p(rb), C.c_int64(N), C.c_int64(d), E, k, _p(w), _ip(i))
    return w, i


def model_forward(mc, tensors, ids, offset=0, causal=True):
    """No-cache forward, logits [B,S,V]."""
    cfg = cfg_of(mc)
    keep, arr = _tensor_array(tensors)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    B, S = ids.shape
    logits = np.empty((B, S, mc.vocab), np.float32)
    lib().orc_model_forward(C.byref(cfg), arr, _ip(ids), C.c_int64(B), C.c_int64(S), C.c_int64(offset), int(bool(causal)),
                            _p(logits))
    return logits


def model_routing(mc, tensors, ids, offset=0, causal=True):
    """The no-cache forward's router decisions: (topi int32, topw f32), each [n_moe_layers, B, S, k]."""
    cfg = cfg_of(mc)
    keep, arr = _tensor_array(tensors)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    B, S = ids.shape
    n_moe = sum(1 for l in range(mc.n_layers) if mc.layer_is_moe(l))
    topi = np.empty((n_moe, B, S, mc.top_k), np.int32)
    topw = np.empty((n_moe, B, S, mc.top_k), np.float32)
    lib().orc_model_routing(C.byref(cfg), arr, _ip(ids), C.c_int64(B), C.c_int64(S), C.c_int64(offset), int(bool(causal)),
                            _ip(topi), _p(topw))
    return topi, topw


def moe_layer(mc, tensors, layer, x):
    cfg = cfg_of(mc)
    keep, arr = _tensor_array(tensors)
    x = _f(x)
    out = np.empty_like(x)
    lib().orc_moe_layer(C.byref(cfg), arr, layer, _p(x), _p(out), C.c_int64(x.shape[0]))
    return out


def generate_greedy(mc, tensors, prompt, n_new, eos=-1, want_all_logits=False):
    """KV-cached greedy generation; returns (ids [B,n_new], last_logits [B,V][, all_logits [n_new,B,V]])."""
    cfg = cfg_of(mc)
    keep, arr = _tensor_array(tensors)
    prompt = np.ascontiguousarray(prompt, dtype=np.int32)
    B, S = prompt.shape
    out = np.empty((B, n_new), np.int32)
    last = np.empty((B, mc.vocab), np.float32)
    alll = np.empty((n_new, B, mc.vocab), np.float32) if want_all_logits else None
    lib().orc_generate_greedy(C.byref(cfg), arr, _ip(prompt), C.c_int64(B), C.c_int64(S), n_new, eos, _ip(out), _p(last),
                              _p(alll) if want_all_logits else None)
    return (out, last, alll) if want_all_logits else (out, last)


FORWARD_FN = C.CFUNCTYPE(None, IP, C.c_int64, C.c_int64, FP, C.c_void_p)


def generate_loop(forward, prompt, vocab, max_new, eos):
    """generate()'s host loop with a Python forward(ids list, offset) -> logits list."""
    def tramp(ids, n, offset, logits_out, user):
        logits = forward([ids[i] for i in range(n)], offset)
        for i, v in enumerate(logits):
            logits_out[i] = v
    cb = FORWARD_FN(tramp)
    prompt = np.ascontiguousarray(prompt, dtype=np.int32)
    toks = np.empty(max_new, np.int32)
    lps = np.empty(max_new, np.float32)
    n = lib().orc_generate_loop(cb, None, _ip(prompt), C.c_int64(prompt.size), C.c_int64(vocab), max_new, eos, _ip(toks),
                                _p(lps))
    return toks[:n].tolist(), lps[:n].tolist()


def decode_bench(mc, tensors, batch, ctx, n_steps):
    """Seconds for n_steps cached decode steps of `batch` sequences at context `ctx`."""
    cfg = cfg_of(mc)
    keep, arr = _tensor_array(tensors)
    last = np.empty(batch, np.int32)
    return float(lib().orc_decode_bench(C.byref(cfg), arr, C.c_int64(batch), C.c_int64(ctx), n_steps, _ip(last)))


# ---- random keys and sampling (src/rew/rng.nim, src/rew/infer/generate.nim:92-150) ----
def threefry(ka, kb, ca, cb):
    out = (C.c_uint32 * 2)()
    lib().orc_threefry(C.c_uint32(ka), C.c_uint32(kb), C.c_uint32(ca), C.c_uint32(cb), out)
    return int(out[0]), int(out[1])


def uniform01(seed, folds=()):
    """uniformF32(key, 1, 0, 1)[0] for key = initKey(seed) folded with each value of `folds` in turn."""
    lib().orc_uniform01.restype = C.c_float
    f = (C.c_uint64 * max(1, len(folds)))(*folds)
    return float(lib().orc_uniform01(C.c_uint64(seed), len(folds), f))


def sample_top_k(logits, top_k, seed):
    lg = _f(logits)
    return int(lib().orc_sample_top_k(_p(lg), C.c_int64(lg.size), int(top_k), C.c_uint64(seed)))


def sample_top_p(logits, top_p, seed):
    lg = _f(logits)
    return int(lib().orc_sample_top_p(_p(lg), C.c_int64(lg.size), C.c_float(top_p), C.c_uint64(seed)))


def generate_sampled(mc, tensors, prompt, n_new, temperature=1.0, top_k=50, top_p=1.0, min_p=0.0,
                     repetition_penalty=1.0, do_sample=True, seeds=None):
    """generate() with a GenerationConfig per sequence of `prompt` [B,S]; returns (ids [B,n_new], logprobs [B,n_new])."""
    cfg = cfg_of(mc)
    keep, arr = _tensor_array(tensors)
    pr = np.ascontiguousarray(prompt, dtype=np.int32)
    if pr.ndim == 1:
        pr = pr.reshape(1, -1)
    B, S = pr.shape
    sd = np.zeros(B, np.uint64) if seeds is None else np.ascontiguousarray(seeds, dtype=np.uint64)
    ids = np.empty((B, n_new), np.int32)
    lps = np.empty((B, n_new), np.float32)
    lib().orc_generate_sampled(C.byref(cfg), arr, _ip(pr), C.c_int64(B), C.c_int64(S), int(n_new), C.c_float(temperature),
                               int(top_k), C.c_float(top_p), C.c_float(min_p), C.c_float(repetition_penalty),
                               int(bool(do_sample)), sd.ctypes.data_as(C.POINTER(C.c_uint64)), _ip(ids), _p(lps))
    return ids, lps


# ---- NF4 codec and QLoRA Linear (src/rew/quantize/codecs.nim:13-74, src/rew/nn/lora.nim:331-431) ----
U8P = C.POINTER(C.c_uint8)


def nf4_quantize(weights, block_size=64):
    """Flat float32 weights -> (packed uint8 [(n+1)//2], scales float32 [ceil(n/block)])."""
    w = _f(weights).reshape(-1)
    n = w.size
    packed = np.zeros((n + 1) // 2, np.uint8)
    scales = np.zeros((n + block_size - 1) // block_size, np.float32)
    lib().orc_nf4_quantize(_p(w), C.c_int64(n), int(block_size), packed.ctypes.data_as(U8P), _p(scales))
    return packed, scales


def nf4_dequantize(packed, scales, n, block_size=64):
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = _f(scales)
    out = np.empty(n, np.float32)
    lib().orc_nf4_dequantize(packed.ctypes.data_as(U8P), _p(scales), C.c_int64(n), int(block_size), _p(out))
    return out


def nf4_roundtrip(w, block_size=64):
    """dequantize(quantize(w)) with w's shape: the frozen base weight a QloraLinear multiplies by."""
    w = _f(w)
    p, s = nf4_quantize(w, block_size)
    return nf4_dequantize(p, s, w.size, block_size).reshape(w.shape)


def qlora_forward(x, packed, scales, n_in, n_out, group_size=64, bias=None, A=None, B=None, scaling=1.0):
    x = _f(x).reshape(-1, n_in)
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = _f(scales)
    rank = 1 if A is None else np.asarray(A).shape[0]
    A = np.zeros((rank, n_in), np.float32) if A is None else _f(A)
    B = np.zeros((n_out, rank), np.float32) if B is None else _f(B)
    b = None if bias is None else _f(bias)
    y = np.empty((x.shape[0], n_out), np.float32)
    lib().orc_qlora_forward(_p(x), C.c_int64(x.shape[0]), packed.ctypes.data_as(U8P), _p(scales), C.c_int64(n_in),
                            C.c_int64(n_out), int(group_size), _p(b) if b is not None else None, _p(A), _p(B), int(rank),
                            C.c_float(scaling), _p(y))
    return y
