"""safetensors reading and the Hugging Face Llama -> rew layout mapping (transpose, rotate-half ->
interleaved RoPE permutation), checked on CPU against a Hugging-Face-convention forward in PyTorch."""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from rew_b200 import safetensors as ST
from rew_b200 import weights as W


def _hf_weights(cfg, seed):
    rng = np.random.default_rng(seed)
    d, hd = cfg.d_model, cfg.head_dim
    t = {"model.embed_tokens.weight": rng.normal(0, 0.05, (cfg.vocab, d)), "model.norm.weight": 1 + 0.1 * rng.normal(size=d),
         "lm_head.weight": rng.normal(0, 0.05, (cfg.vocab, d))}
    for l in range(cfg.n_layers):
        p = "model.layers.%d." % l
        t[p + "self_attn.q_proj.weight"] = rng.normal(0, 0.05, (cfg.n_heads * hd, d))
        t[p + "self_attn.k_proj.weight"] = rng.normal(0, 0.05, (cfg.n_kv_heads * hd, d))
        t[p + "self_attn.v_proj.weight"] = rng.normal(0, 0.05, (cfg.n_kv_heads * hd, d))
        t[p + "self_attn.o_proj.weight"] = rng.normal(0, 0.05, (d, cfg.n_heads * hd))
        def ffn(prefix, width):
            t[prefix + "gate_proj.weight"] = rng.normal(0, 0.05, (width, d))
            t[prefix + "up_proj.weight"] = rng.normal(0, 0.05, (width, d))
            t[prefix + "down_proj.weight"] = rng.normal(0, 0.05, (d, width))

        if cfg.layer_is_moe(l):     # DeepSeek-MoE naming: router, one fused shared FFN, routed experts
            t[p + "mlp.gate.weight"] = rng.normal(0, 0.5, (cfg.n_routed, d))
            ffn(p + "mlp.shared_experts.", cfg.n_shared * cfg.moe_ffn)
            for e in range(cfg.n_routed):
                ffn(p + "mlp.experts.%d." % e, cfg.moe_ffn)
        else:
            ffn(p + "mlp.", cfg.first_dense if cfg.n_routed > 0 and cfg.first_dense > 0 else cfg.ffn)
        t[p + "input_layernorm.weight"] = 1 + 0.1 * rng.normal(size=d)
        t[p + "post_attention_layernorm.weight"] = 1 + 0.1 * rng.normal(size=d)
    return {k: v.astype(np.float32) for k, v in t.items()}


def _hf_forward(cfg, t, ids):
    """Llama as Hugging Face computes it: x @ W.T, RMSNorm, rotate-half RoPE, causal attention."""
    P = {k: torch.from_numpy(v.astype(np.float64)) for k, v in t.items()}
    B, S = ids.shape
    hd, nh, kvh = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    inv = 1.0 / (cfg.theta ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    ang = torch.arange(S, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)

    def rot(x):
        x1, x2 = x[..., :hd // 2], x[..., hd // 2:]
        return x * cos + torch.cat([-x2, x1], -1) * sin

    def rms(x, g):
        return g * (x / torch.sqrt((x * x).mean(-1, keepdim=True) + cfg.eps))

    h = P["model.embed_tokens.weight"][torch.from_numpy(ids).long()]
    mask = torch.triu(torch.full((S, S), float("-inf"), dtype=torch.float64), 1)
    for l in range(cfg.n_layers):
        p = "model.layers.%d." % l
        x = rms(h, P[p + "input_layernorm.weight"])
        q = (x @ P[p + "self_attn.q_proj.weight"].T).view(B, S, nh, hd).transpose(1, 2)
        k = (x @ P[p + "self_attn.k_proj.weight"].T).view(B, S, kvh, hd).transpose(1, 2)
        v = (x @ P[p + "self_attn.v_proj.weight"].T).view(B, S, kvh, hd).transpose(1, 2)
        q, k = rot(q), rot(k)
        k, v = k.repeat_interleave(nh // kvh, 1), v.repeat_interleave(nh // kvh, 1)
        a = torch.softmax(q @ k.transpose(-1, -2) / np.sqrt(hd) + mask, -1) @ v
        h = h + a.transpose(1, 2).reshape(B, S, nh * hd) @ P[p + "self_attn.o_proj.weight"].T
        x = rms(h, P[p + "post_attention_layernorm.weight"])
        def ffn(prefix, xx):
            g, u = xx @ P[prefix + "gate_proj.weight"].T, xx @ P[prefix + "up_proj.weight"].T
            return (torch.nn.functional.silu(g) * u) @ P[prefix + "down_proj.weight"].T

        if cfg.layer_is_moe(l):     # softmax gate, top-k, renormalised weights, plus the shared FFN
            scores = torch.softmax(x @ P[p + "mlp.gate.weight"].T, -1)
            topw, topi = scores.topk(cfg.top_k, -1)
            topw = topw / topw.sum(-1, keepdim=True)
            y = ffn(p + "mlp.shared_experts.", x)
            for e in range(cfg.n_routed):
                we = (topw * (topi == e)).sum(-1, keepdim=True)
                y = y + we * ffn(p + "mlp.experts.%d." % e, x)
            h = h + y
        else:
            h = h + ffn(p + "mlp.", x)
    return (rms(h, P["model.norm.weight"]) @ P["lm_head.weight"].T).numpy()


def test_safetensors_round_trip(tmp_path):
    cfg = W.tiny_llama(mask_kind=1)
    t = _hf_weights(cfg, 0)
    ST.write_safetensors(str(tmp_path / "m.safetensors"), t)
    back = ST.read_safetensors(str(tmp_path / "m.safetensors"))
    assert set(back) == set(t) and all(np.array_equal(back[k], t[k]) for k in t)
    ST.write_safetensors(str(tmp_path / "b.safetensors"), t, dtype="BF16")
    back = ST.read_safetensors(str(tmp_path / "b.safetensors"))
    assert all(np.array_equal(back[k], W.bf16_round(t[k])) for k in t)


def test_hf_llama_mapping_reproduces_hf_semantics(tmp_path, orc):
    cfg = W.tiny_llama(mask_kind=1, norm_kind=0)
    t = _hf_weights(cfg, 1)
    ST.write_safetensors(str(tmp_path / "m.safetensors"), t)
    canon = ST.llama_from_hf(cfg, ST.read_safetensors(str(tmp_path / "m.safetensors")))
    ids = np.random.default_rng(2).integers(0, cfg.vocab, size=(2, 12)).astype(np.int32)
    got = orc.model_forward(cfg, canon, ids, 0, True)     # rew semantics on the converted weights
    want = _hf_forward(cfg, t, ids)                       # Hugging Face semantics on the original ones
    assert rel_l2(got, want) < 5e-6
    # tied head when lm_head.weight is absent
    t2 = {k: v for k, v in t.items() if k != "lm_head.weight"}
    canon2 = ST.llama_from_hf(cfg, t2)
    assert np.array_equal(canon2[-2], t["model.embed_tokens.weight"].T)


def test_hf_deepseek_moe_mapping_reproduces_hf_semantics(orc):
    """DeepSeek-MoE naming (standard attention, mlp.gate / mlp.experts.N / one fused mlp.shared_experts,
    dense first layer) mapped onto rew's DeepSeekMoE tensors (src/rew/models/deepseek.nim:36-63)."""
    cfg = W.ModelConfig(vocab=96, d_model=64, n_layers=3, n_heads=4, n_kv_heads=4, head_dim=16, ffn=0, max_seq=64,
                        theta=10000.0, eps=1e-6, norm_kind=0, mask_kind=1, n_routed=6, n_shared=2, top_k=2, moe_ffn=48,
                        first_dense=80)
    t = _hf_weights(cfg, 5)
    canon = ST.llama_from_hf(cfg, t)
    assert len(canon) == len(W.tensor_specs(cfg))
    ids = np.random.default_rng(6).integers(0, cfg.vocab, size=(2, 9)).astype(np.int32)
    got = orc.model_forward(cfg, canon, ids, 0, True)
    want = _hf_forward(cfg, t, ids)
    assert rel_l2(got, want) < 5e-6


def test_sharded_snapshot_directory_and_hf_config(tmp_path, orc):
    """A checkpoint split over several *.safetensors shards plus its config.json loads to the same canonical
    tensors as the single file; a tensor present in two shards is refused; absent config keys take the
    reference's defaults (src/rew/hf/hub.nim:370-382)."""
    import json
    cfg = W.tiny_llama(mask_kind=1, norm_kind=0)
    t = _hf_weights(cfg, 3)
    names = sorted(t)
    snap = tmp_path / "snap"
    snap.mkdir()
    third = (len(names) + 2) // 3
    for i in range(3):
        part = {k: t[k] for k in names[i * third:(i + 1) * third]}
        ST.write_safetensors(str(snap / ("model-%05d-of-00003.safetensors" % (i + 1))), part, dtype="BF16" if i == 1 else "F32")
    (snap / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {}}))
    hf_cfg = {"vocab_size": cfg.vocab, "hidden_size": cfg.d_model, "intermediate_size": cfg.ffn,
              "num_hidden_layers": cfg.n_layers, "num_attention_heads": cfg.n_heads,
              "num_key_value_heads": cfg.n_kv_heads, "max_position_embeddings": cfg.max_seq,
              "rope_theta": cfg.theta, "rms_norm_eps": cfg.eps, "architectures": ["LlamaForCausalLM"]}
    (snap / "config.json").write_text(json.dumps(hf_cfg))
    got_cfg = ST.llama_config_from_hf(str(snap / "config.json"))
    for f in ("vocab", "d_model", "n_layers", "n_heads", "n_kv_heads", "head_dim", "ffn", "max_seq", "theta", "eps"):
        assert getattr(got_cfg, f) == getattr(cfg, f), f
    merged = ST.read_safetensors_dir(str(snap))
    assert set(merged) == set(t)
    want = {k: (W.bf16_round(t[k]) if k in names[third:2 * third] else t[k]) for k in t}
    assert all(np.array_equal(merged[k], want[k]) for k in t)
    canon = ST.llama_from_hf(got_cfg, merged)
    ref = ST.llama_from_hf(cfg, want)
    assert all(np.array_equal(a, b) for a, b in zip(canon, ref))
    # defaults of toLlamaConfig
    d = ST.llama_config_from_hf({})
    assert (d.vocab, d.d_model, d.ffn, d.n_layers, d.n_heads, d.n_kv_heads, d.max_seq, d.theta) == \
           (32000, 4096, 11008, 32, 32, 32, 2048, 10000.0)
    assert ST.llama_config_from_hf({"num_attention_heads": 8, "hidden_size": 512}).n_kv_heads == 8
    # the same tensor in two shards is an error
    ST.write_safetensors(str(snap / "zz-extra.safetensors"), {names[0]: t[names[0]]})
    with pytest.raises(ValueError, match="more than one shard"):
        ST.read_safetensors_dir(str(snap))
    with pytest.raises(FileNotFoundError):
        ST.read_safetensors_dir(str(tmp_path))


def test_config_keys_that_change_the_model_are_refused():
    """toLlamaConfig (src/rew/hf/hub.nim:370-382) ignores rope_scaling and head_dim; a checkpoint that sets them
    would load and then compute another model's logits, so the loader refuses instead."""
    base = {"num_attention_heads": 8, "hidden_size": 512}
    with pytest.raises(ValueError, match="rope_scaling"):
        ST.llama_config_from_hf(dict(base, rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}))
    with pytest.raises(ValueError, match="rope_scaling"):
        ST.llama_config_from_hf(dict(base, rope_scaling={"type": "linear", "factor": 2.0}))
    with pytest.raises(ValueError, match="head_dim"):
        ST.llama_config_from_hf(dict(base, head_dim=128))
    assert ST.llama_config_from_hf(dict(base, rope_scaling=None, head_dim=64)).head_dim == 64
    assert ST.llama_config_from_hf(dict(base, rope_scaling={"rope_type": "default"})).head_dim == 64


def test_byte_ranges_are_checked_for_every_dtype(tmp_path):
    import json
    import struct
    for dt, itemsize in (("BF16", 2), ("F16", 2), ("F64", 8), ("F32", 4)):
        header = {"w": {"dtype": dt, "shape": [4, 4], "data_offsets": [0, 16 * itemsize - itemsize]}}  # one element short
        hj = json.dumps(header).encode()
        hj += b" " * ((8 - len(hj) % 8) % 8)
        path = tmp_path / ("bad_%s.safetensors" % dt)
        path.write_bytes(struct.pack("<Q", len(hj)) + hj + b"\0" * (16 * itemsize))
        with pytest.raises(ValueError, match="inconsistent offsets"):
            ST.read_safetensors(str(path))
    header = {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 64]}}
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    (tmp_path / "oob.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"\0" * 16)
    with pytest.raises(ValueError, match="outside the file"):
        ST.read_safetensors(str(tmp_path / "oob.safetensors"))
