"""safetensors files and the Hugging Face Llama naming → this backend's canonical tensors.

File format as rew reads it (src/rew/safetensors.nim:1-80): 8-byte little-endian header length, a JSON
header {name: {"dtype", "shape", "data_offsets": [start, end]}, "__metadata__": {...}}, then the raw
tensor bytes.  rew's own loadLlamaWeights (src/rew/hf/hub.nim:395-430) walks the Hugging Face names but
discards every tensor; this module does the mapping that stub leaves out:

  * HF Linear weights are [out, in]; rew's are [in, out] (src/rew/nn/linear.nim:21-25): transpose.
  * HF Llama applies RoPE to the pairs (i, i + head_dim/2) ("rotate half"); rew rotates the interleaved
    pairs (2i, 2i+1) (src/rew/nn/rope.nim:56-108).  Permuting the output features of q_proj and k_proj
    inside every head (rew feature 2i <- HF i, 2i+1 <- HF i + head_dim/2) makes the two equivalent:
    scores are dot products over the head dimension, so a common permutation of q and k cancels.
  * RMSNorm weights become gamma with beta = 0 (use norm_kind = 0); missing biases are zero; a missing
    lm_head.weight is tied to the embedding.
"""
import json
import struct

import numpy as np

from .weights import from_bf16_bits, tensor_specs, to_bf16_bits

_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I32": np.int32, "I64": np.int64, "U8": np.uint8,
           "I8": np.int8, "I16": np.int16, "BOOL": np.bool_}


def read_safetensors(path):
    """{name: float32/int numpy array}; BF16 and F16 are widened to float32."""
    with open(path, "rb") as f:
        raw = f.read()
    if len(raw) < 8:
        raise ValueError("safetensors: file too short")
    (hlen,) = struct.unpack("<Q", raw[:8])
    if 8 + hlen > len(raw):
        raise ValueError("safetensors: header length exceeds the file")
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    data = memoryview(raw)[8 + hlen:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        start, end = info["data_offsets"]
        shape = tuple(info["shape"])
        if not (0 <= start <= end <= len(data)):
            raise ValueError("safetensors: tensor %s has offsets outside the file" % name)
        buf = data[start:end]
        dt = info["dtype"]
        itemsize = 2 if dt == "BF16" else (np.dtype(_DTYPES[dt]).itemsize if dt in _DTYPES else None)
        if itemsize is None:
            raise ValueError("unsupported safetensors dtype: " + dt)
        numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if end - start != numel * itemsize:      # every dtype: the byte range must hold exactly the declared shape
            raise ValueError("safetensors: tensor %s has inconsistent offsets (%d bytes for shape %r of %s)"
                             % (name, end - start, shape, dt))
        if dt == "BF16":
            arr = from_bf16_bits(np.frombuffer(buf, dtype=np.uint16)).reshape(shape)
        else:
            arr = np.frombuffer(buf, dtype=_DTYPES[dt]).reshape(shape)
            if dt in ("F16", "F64"):
                arr = arr.astype(np.float32)
        out[name] = arr
    return out


def read_safetensors_dir(snap_dir):
    """loadSafetensorsWeights (src/rew/hf/hub.nim:386-394): every *.safetensors file of a snapshot directory
    merged into one {name: array}, which covers single-file and sharded checkpoints alike (the shard index
    model.safetensors.index.json is not needed: each shard names its own tensors).  Files are visited in
    sorted order; a tensor named by two shards is an error rather than a silent overwrite."""
    import glob
    import os
    files = sorted(f for f in glob.glob(os.path.join(snap_dir, "*.safetensors")) if not f.endswith(".index.json"))
    if not files:
        raise FileNotFoundError("no *.safetensors file in %s" % snap_dir)
    out = {}
    for f in files:
        for name, arr in read_safetensors(f).items():
            if name in out:
                raise ValueError("tensor %s appears in more than one shard of %s" % (name, snap_dir))
            out[name] = arr
    return out


def llama_config_from_hf(path_or_dict, dtype=None, **overrides):
    """loadHfConfig + toLlamaConfig (src/rew/hf/hub.nim:344-382): a Hugging Face config.json -> ModelConfig, with
    the reference's defaults for absent keys (vocab 32000, hidden 4096, intermediate 11008, 32 layers, 32 heads,
    kv heads = heads, 2048 positions, rope_theta 10000, rms_norm_eps 1e-5).  head_dim is hidden / heads as in
    initLlamaConfig; norm_kind 0 (RMSNorm weights) and the conventional causal mask are what a Hugging Face
    checkpoint means."""
    from .weights import ModelConfig
    node = path_or_dict
    if not isinstance(node, dict):
        with open(path_or_dict) as f:
            node = json.load(f)
    heads = int(node.get("num_attention_heads", 32))
    hidden = int(node.get("hidden_size", 4096))
    # toLlamaConfig reads neither key; a checkpoint that sets them means another model than the one built here
    # (Llama-3.1 style frequency scaling changes every RoPE angle; an explicit head_dim decouples it from
    # hidden / heads), so loading it silently would give wrong logits.
    scaling = node.get("rope_scaling")
    if scaling is not None and not (isinstance(scaling, dict) and scaling.get("rope_type", scaling.get("type")) in (None, "default")):
        raise ValueError("config.json: rope_scaling %r is not supported (initRotaryPositionEncoding has plain RoPE only, "
                         "src/rew/nn/rope.nim:112-145)" % (scaling,))
    if node.get("head_dim") is not None and int(node["head_dim"]) != hidden // heads:
        raise ValueError("config.json: head_dim %r differs from hidden_size / num_attention_heads = %d, which "
                         "initLlamaConfig assumes" % (node["head_dim"], hidden // heads))
    kw = dict(vocab=int(node.get("vocab_size", 32000)), d_model=hidden, n_layers=int(node.get("num_hidden_layers", 32)),
              n_heads=heads, n_kv_heads=int(node.get("num_key_value_heads", heads)), head_dim=hidden // heads,
              ffn=int(node.get("intermediate_size", 11008)), max_seq=int(node.get("max_position_embeddings", 2048)),
              theta=float(node.get("rope_theta", 10000.0)), eps=float(node.get("rms_norm_eps", 1e-5)),
              norm_kind=0, mask_kind=1)
    if dtype is not None:
        kw["dtype"] = dtype
    kw.update(overrides)
    return ModelConfig(**kw)


def write_safetensors(path, tensors, dtype="F32"):
    """Writes {name: array}; dtype F32 or BF16 for floating tensors."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        if a.dtype == np.float32 and dtype == "BF16":
            blob, dt = to_bf16_bits(a).tobytes(), "BF16"
        else:
            blob = a.tobytes()
            dt = {np.dtype(np.float32): "F32", np.dtype(np.int32): "I32", np.dtype(np.int64): "I64"}[a.dtype]
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(blob)]}
        blobs.append(blob)
        off += len(blob)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def _interleave_heads(w_out_in, n_heads, head_dim):
    """Reorders output features (axis 0 of an HF [out, in] weight, or a bias) inside each head from the
    rotate-half layout to rew's interleaved layout."""
    half = head_dim // 2
    perm = np.empty(head_dim, np.int64)
    perm[0::2] = np.arange(half)
    perm[1::2] = np.arange(half) + half
    idx = (np.arange(n_heads)[:, None] * head_dim + perm[None, :]).ravel()
    return w_out_in[idx]


def llama_from_hf(cfg, hf):
    """Canonical tensor list (rew_b200.weights.tensor_specs order) from Hugging Face Llama tensors, or from a
    DeepSeek-MoE checkpoint with standard attention (q_proj / k_proj / v_proj / o_proj; MoE blocks named
    mlp.gate, mlp.experts.N, mlp.shared_experts) when cfg.n_routed > 0."""
    d, hd = cfg.d_model, cfg.head_dim

    def get(name, default=None):
        if name in hf:
            return np.asarray(hf[name], np.float32)
        if default is None:
            raise KeyError("safetensors: missing tensor " + name)
        return default

    out = {}
    embed = get("model.embed_tokens.weight")
    out["model.embedTokens.weight"] = embed
    for l in range(cfg.n_layers):
        hp, p = "model.layers.%d." % l, "model.layers.%d." % l
        for hf_name, name, heads in (("q_proj", "qProj", cfg.n_heads), ("k_proj", "kProj", cfg.n_kv_heads),
                                     ("v_proj", "vProj", 0), ("o_proj", "outProj", 0)):
            w = get(hp + "self_attn.%s.weight" % hf_name)                       # [out, in]
            b = get(hp + "self_attn.%s.bias" % hf_name, np.zeros(w.shape[0], np.float32))
            if heads:
                w, b = _interleave_heads(w, heads, hd), _interleave_heads(b, heads, hd)
            out[p + "selfAttn.%s.weight" % name] = np.ascontiguousarray(w.T)      # [in, out]
            out[p + "selfAttn.%s.bias" % name] = b
        def ffn(dst, src, rows=None):
            """One gated FFN: HF [out,in] -> [in,out]; `rows` selects a slice of the hidden width."""
            for hf_name, name in (("gate_proj", "gateProj"), ("up_proj", "upProj"), ("down_proj", "downProj")):
                w = get(src + "%s.weight" % hf_name)
                if rows is not None:
                    w = w[:, rows] if hf_name == "down_proj" else w[rows]
                out[dst + "%s.weight" % name] = np.ascontiguousarray(w.T)
                b = hf.get(src + "%s.bias" % hf_name)
                if b is not None and rows is not None:
                    if hf_name != "down_proj":
                        b = np.asarray(b, np.float32)[rows]
                    elif rows.start != 0:
                        b = None                                                 # the fused FFN's output bias counts once
                out[dst + "%s.bias" % name] = np.zeros(w.shape[0], np.float32) if b is None else np.asarray(b, np.float32)

        if cfg.layer_is_moe(l):
            # DeepSeekMoE (src/rew/models/deepseek.nim:36-63): router Linear, shared experts, routed experts.
            # Hugging Face stores the shared experts as ONE FFN of width n_shared * moe_ffn; a sum of FFNs
            # over disjoint slices of the hidden width is the same function.
            f = cfg.moe_ffn
            gw = get(hp + "mlp.gate.weight")                                         # [n_routed, d]
            out[p + "moe.gate.weight"] = np.ascontiguousarray(gw.T)
            out[p + "moe.gate.bias"] = np.zeros(cfg.n_routed, np.float32)
            for e in range(cfg.n_shared):
                ffn(p + "moe.sharedExperts.%d." % e, hp + "mlp.shared_experts.", slice(e * f, (e + 1) * f))
            for e in range(cfg.n_routed):
                ffn(p + "moe.routedExperts.%d." % e, hp + "mlp.experts.%d." % e)
        else:
            ffn(p + "mlp.", hp + "mlp.")
        out[p + "inputLayernorm.gamma"] = get(hp + "input_layernorm.weight")
        out[p + "inputLayernorm.beta"] = np.zeros(d, np.float32)
        out[p + "postAttentionLayernorm.gamma"] = get(hp + "post_attention_layernorm.weight")
        out[p + "postAttentionLayernorm.beta"] = np.zeros(d, np.float32)
    out["model.norm.gamma"] = get("model.norm.weight")
    out["model.norm.beta"] = np.zeros(d, np.float32)
    lm = get("lm_head.weight", embed)                                            # tied when absent
    out["lmHead.weight"] = np.ascontiguousarray(lm.T)
    out["lmHead.bias"] = np.zeros(cfg.vocab, np.float32)
    specs = tensor_specs(cfg)
    for name, shape in specs:
        if tuple(out[name].shape) != tuple(shape):
            raise ValueError("safetensors: %s has shape %r, expected %r" % (name, out[name].shape, shape))
    return [out[name] for name, _ in specs]
