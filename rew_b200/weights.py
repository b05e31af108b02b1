"""Model configurations and the canonical order of a model's logical tensors.

The order is the one rewb200_model_set_tensor indexes by.  Names follow rew's pytree fields
(src/rew/models/llama.nim:27-44, src/rew/models/deepseek.nim:36-63).
"""
from dataclasses import dataclass, asdict

import numpy as np

from . import _lib


@dataclass
class ModelConfig:
    vocab: int
    d_model: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    max_seq: int = 2048
    theta: float = 10000.0
    eps: float = 1e-5
    norm_kind: int = 0      # 0: rmsNorm math; 1: LayerNorm as LlamaDecoderLayer is written
    mask_kind: int = 0      # 0: makeCausalMask as written; 1: conventional causal
    n_routed: int = 0
    n_shared: int = 0
    top_k: int = 0
    moe_ffn: int = 0
    first_dense: int = 0
    dtype: int = _lib.F32
    tp_rank: int = 0
    tp_size: int = 1
    ep_rank: int = 0
    ep_size: int = 1
    weight_quant: int = 0   # 1: decoder Linear weights as NF4 codes (blocks of 64) on the device

    def to_c(self):
        return _lib.Config(**asdict(self))

    def layer_is_moe(self, l):
        return self.n_routed > 0 and not (self.first_dense > 0 and l == 0)


# Benchmark configurations (shapes only; weights are synthetic).
def tiny_llama(**kw):
    return ModelConfig(vocab=1024, d_model=256, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=32, ffn=688,
                       max_seq=128, theta=10000.0, eps=1e-5, **kw)


def llama3_8b(**kw):
    return ModelConfig(vocab=128256, d_model=4096, n_layers=32, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336,
                       max_seq=2048, theta=500000.0, eps=1e-5, dtype=_lib.BF16, mask_kind=1, **kw)


def llama3_70b(**kw):
    return ModelConfig(vocab=128256, d_model=8192, n_layers=80, n_heads=64, n_kv_heads=8, head_dim=128, ffn=28672,
                       max_seq=2048, theta=500000.0, eps=1e-5, dtype=_lib.BF16, mask_kind=1, **kw)


def deepseek_v2_lite(**kw):
    return ModelConfig(vocab=102400, d_model=2048, n_layers=27, n_heads=16, n_kv_heads=16, head_dim=128, ffn=10944,
                       max_seq=1024, theta=10000.0, eps=1e-6, n_routed=64, n_shared=2, top_k=6, moe_ffn=1408,
                       first_dense=10944, dtype=_lib.BF16, mask_kind=1, **kw)


def tensor_specs(cfg):
    """[(name, shape)] in canonical order; every Linear is weight [in,out] then bias [out]."""
    d, hd = cfg.d_model, cfg.head_dim
    nq, nkv = cfg.n_heads * hd, cfg.n_kv_heads * hd
    specs = [("model.embedTokens.weight", (cfg.vocab, d))]

    def lin(prefix, i, o):
        return [(prefix + ".weight", (i, o)), (prefix + ".bias", (o,))]

    def ffn(prefix, width):
        return lin(prefix + ".gateProj", d, width) + lin(prefix + ".upProj", d, width) + lin(prefix + ".downProj", width, d)

    for l in range(cfg.n_layers):
        p = "model.layers.%d" % l
        specs += [(p + ".inputLayernorm.gamma", (d,)), (p + ".inputLayernorm.beta", (d,))]
        specs += lin(p + ".selfAttn.qProj", d, nq) + lin(p + ".selfAttn.kProj", d, nkv)
        specs += lin(p + ".selfAttn.vProj", d, nkv) + lin(p + ".selfAttn.outProj", nq, d)
        specs += [(p + ".postAttentionLayernorm.gamma", (d,)), (p + ".postAttentionLayernorm.beta", (d,))]
        if cfg.layer_is_moe(l):
            specs += lin(p + ".moe.gate", d, cfg.n_routed)
            for e in range(cfg.n_shared):
                specs += ffn(p + ".moe.sharedExperts.%d" % e, cfg.moe_ffn)
            for e in range(cfg.n_routed):
                specs += ffn(p + ".moe.routedExperts.%d" % e, cfg.moe_ffn)
        else:
            width = cfg.first_dense if (cfg.n_routed > 0 and cfg.first_dense > 0) else cfg.ffn
            specs += ffn(p + ".mlp", width)
    specs += [("model.norm.gamma", (d,)), ("model.norm.beta", (d,))]
    specs += lin("lmHead", d, cfg.vocab)
    return specs


def init_weights(cfg, seed=0, std=0.02, trivial_affine=True):
    """Seeded synthetic tensors in canonical order.

    Matrices ~ N(0, std) drawn in canonical order from numpy's default_rng(seed).
    With trivial_affine (the reference's init: src/rew/nn/linear.nim:37,
    src/rew/nn/norm.nim:30-38) biases are 0, gammas 1, betas 0; otherwise they
    are small random values so tests exercise those terms too.
    """
    rng = np.random.default_rng(seed)
    out = []
    for name, shape in tensor_specs(cfg):
        if len(shape) == 2:
            t = rng.normal(0.0, std, size=shape).astype(np.float32)
        elif trivial_affine:
            t = np.ones(shape, np.float32) if name.endswith("gamma") else np.zeros(shape, np.float32)
        else:
            base = 1.0 if name.endswith("gamma") else 0.0
            t = (base + rng.normal(0.0, 0.05, size=shape)).astype(np.float32)
        out.append(t)
    return out


def bf16_round(x):
    """Round-to-nearest-even of f32 values to bf16 precision, kept as f32
    (src/rew/ops/literal.nim:112-116)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    bits = bits + 0x7FFF + ((bits >> 16) & 1)
    return ((bits & 0xFFFF0000).astype(np.uint32)).view(np.float32).reshape(x.shape)


def to_bf16_bits(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    bits = bits + 0x7FFF + ((bits >> 16) & 1)
    return (bits >> 16).astype(np.uint16).reshape(x.shape)


def from_bf16_bits(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32).reshape(b.shape)
