"""CPU tests of the oracle: the reference's own known-answer vectors for the
primitives and the generate loop, known-answer properties for the layers the
reference never pins, an independent PyTorch restatement, and the committed
golden fixtures."""
import os

import numpy as np
import pytest
import torch

from conftest import rel_l2
from rew_b200 import weights as W

GOLD = os.path.join(os.path.dirname(__file__), "golden")


# ---- vectors from the reference's tests/teager_dispatch.nim -------------------
A = np.array([1, 2, 3, 4], np.float32)
B = np.array([10, 20, 30, 40], np.float32)


def test_pin_add_mul_neg(orc):  # teager_dispatch.nim:264-284
    assert orc.binary("add", A, B).tolist() == [11.0, 22.0, 33.0, 44.0]
    assert orc.binary("mul", A, B).tolist() == [10.0, 40.0, 90.0, 160.0]
    assert orc.unary("neg", A).tolist() == [-1.0, -2.0, -3.0, -4.0]


def test_pin_exp_logistic(orc):  # teager_dispatch.nim:286-291,338-343
    got = orc.unary("exp", A)
    for i, v in enumerate(got):
        assert abs(v - np.exp(np.float32(i + 1))) < 1e-5 * max(1.0, v)
    got = orc.unary("logistic", A)
    for i, v in enumerate(got):
        assert abs(v - 1.0 / (1.0 + np.exp(-np.float32(i + 1)))) < 1e-4


def test_pin_matmul_reduce_transpose_iota(orc):  # teager_dispatch.nim:584-598,562-566,549-554,505-509
    assert orc.matmul(A.reshape(2, 2), B.reshape(2, 2)).ravel().tolist() == [70.0, 100.0, 150.0, 220.0]
    assert orc.reduce_sum(A) == 10.0
    assert orc.transpose2d(A.reshape(2, 2)).ravel().tolist() == [1.0, 3.0, 2.0, 4.0]
    assert orc.iota2d(2, 3, 1).ravel().tolist() == [0, 1, 2, 0, 1, 2]


def test_pin_generate_loop(orc):  # tests/tgenerate.nim:21-52
    calls = {"n": 0, "offsets": [], "inputs": []}

    def forward(ids, offset):
        calls["offsets"].append(offset)
        calls["inputs"].append(list(ids))
        nxt = 4 if calls["n"] == 0 else 2
        calls["n"] += 1
        logits = [-10.0] * 5
        logits[nxt] = 10.0
        return logits

    toks, lps = orc.generate_loop(forward, [7, 8, 9], vocab=5, max_new=3, eos=2)
    assert [7, 8, 9] + toks == [7, 8, 9, 4, 2]
    assert len(lps) == 2
    assert calls["offsets"] == [0, 3]
    assert calls["inputs"] == [[7, 8, 9], [4]]


def test_bf16_round_matches_bit_formula(orc):  # src/rew/ops/literal.nim:112-116
    x = np.random.default_rng(0).normal(size=1000).astype(np.float32)
    got = orc.bf16_round(x)
    assert np.array_equal(got, W.bf16_round(x))
    assert np.array_equal(got, torch.from_numpy(x).to(torch.bfloat16).float().numpy())


# ---- known answers the reference never pins -----------------------------------
def test_rope_identity_at_pos0_and_rotation_at_pos1(orc):
    c, s = orc.rope_tables(2, 4, 10000.0)
    x = np.array([[[3.0, 4.0], [3.0, 4.0]]], np.float32)  # [1, S=2, hd=2]
    y = orc.rope_apply(x, c, s, 0)
    assert np.array_equal(y[0, 0], x[0, 0])  # angle 0
    c1, s1 = np.float32(np.cos(np.float32(1.0))), np.float32(np.sin(np.float32(1.0)))
    np.testing.assert_allclose(y[0, 1], [c1 * 3 - s1 * 4, s1 * 3 + c1 * 4], rtol=1e-6)
    # tables hold each value twice (rope.nim:134-138)
    c8, s8 = orc.rope_tables(8, 16, 500000.0)
    assert np.array_equal(c8[:, 0::2], c8[:, 1::2]) and np.array_equal(s8[:, 0::2], s8[:, 1::2])
    # the offset shifts table rows
    x2 = np.random.default_rng(1).normal(size=(2, 5, 8)).astype(np.float32)
    full = orc.rope_apply(np.concatenate([np.zeros((2, 3, 8), np.float32), x2], 1), c8, s8, 0)[:, 3:]
    assert np.array_equal(orc.rope_apply(x2, c8, s8, 3), full)


def test_softmax_rows_sum_to_one(orc):
    x = np.random.default_rng(2).normal(size=(7, 33)).astype(np.float32) * 5
    p = orc.softmax(x)
    np.testing.assert_allclose(p.sum(-1), 1.0, rtol=1e-6)
    assert (p >= 0).all()


def test_mask_variants_are_transposes(orc):
    a, b = orc.causal_mask(6, 6, 0), orc.causal_mask(6, 6, 1)
    assert np.array_equal(a, b.T)
    assert a[0, 5] == 0 and a[5, 0] == np.float32(-1e9)  # as written: query i sees keys j >= i


def test_gqa_equals_mha_when_heads_match(orc):
    rng = np.random.default_rng(3)
    q = rng.normal(size=(2, 4, 5, 8)).astype(np.float32)
    k = rng.normal(size=(2, 2, 5, 8)).astype(np.float32)
    v = rng.normal(size=(2, 2, 5, 8)).astype(np.float32)
    got = orc.gqa_attention(q, k, v, True, 1)
    want = orc.gqa_attention(q, np.repeat(k, 2, 1), np.repeat(v, 2, 1), True, 1)
    assert np.array_equal(got, want)


def test_gather_equals_onehot_matmul(orc):
    rng = np.random.default_rng(4)
    table = rng.normal(size=(50, 12)).astype(np.float32)
    ids = rng.integers(0, 50, size=(9,)).astype(np.int32)
    assert np.array_equal(orc.embedding_onehot(ids, table), table[ids])


def test_cached_decode_equals_recompute_under_standard_mask(orc):
    cfg = W.tiny_llama(mask_kind=1)
    t = W.init_weights(cfg, seed=3, trivial_affine=False)
    prompt = np.random.default_rng(5).integers(0, cfg.vocab, size=(2, 9)).astype(np.int32)
    ids, last, alll = orc.generate_greedy(cfg, t, prompt, 4, want_all_logits=True)
    seq = np.concatenate([prompt, ids[:, :3]], 1)
    full = orc.model_forward(cfg, t, seq, 0, True)
    for step in range(4):
        np.testing.assert_allclose(alll[step], full[:, 8 + step], rtol=2e-5, atol=2e-6)


def test_moe_sparse_equals_dense_all_experts(orc):
    cfg = W.ModelConfig(vocab=64, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=8, ffn=48, max_seq=32,
                        n_routed=8, n_shared=2, top_k=3, moe_ffn=16, first_dense=48)
    t = W.init_weights(cfg, seed=6, std=0.3)
    specs = W.tensor_specs(cfg)
    x = np.random.default_rng(7).normal(size=(5, 32)).astype(np.float32)
    got = orc.moe_layer(cfg, t, 1, x)
    # dense restatement in numpy, every expert on every token (deepseek.nim:140-144)
    names = [n for n, _ in specs]
    def T(n):
        return t[names.index("model.layers.1.moe." + n)].astype(np.float64)
    def ffn(prefix, xx):
        g = xx @ T(prefix + ".gateProj.weight") + T(prefix + ".gateProj.bias")
        u = xx @ T(prefix + ".upProj.weight") + T(prefix + ".upProj.bias")
        return (g / (1 + np.exp(-g)) * u) @ T(prefix + ".downProj.weight") + T(prefix + ".downProj.bias")
    xx = x.astype(np.float64)
    out = sum(ffn("sharedExperts.%d" % e, xx) for e in range(2))
    logits = xx @ T("gate.weight") + T("gate.bias")
    p = np.exp(logits - logits.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    top = np.argsort(-p, -1, kind="stable")[:, :3]
    wts = np.take_along_axis(p, top, -1)
    wts /= wts.sum(-1, keepdims=True)
    for e in range(8):
        w_e = (wts * (top == e)).sum(-1)
        out = out + ffn("routedExperts.%d" % e, xx) * w_e[:, None]
    np.testing.assert_allclose(got, out, rtol=1e-4, atol=1e-5)
    tw, ti = orc.moe_route(x, t[names.index("model.layers.1.moe.gate.weight")], t[names.index("model.layers.1.moe.gate.bias")], 3)
    assert np.array_equal(ti, top.astype(np.int32))
    np.testing.assert_allclose(tw.sum(-1), 1.0, rtol=1e-6)


# ---- independent restatement in PyTorch (CPU, float64) ------------------------
def _torch_forward(cfg, tensors, ids, offset, causal):
    names = [n for n, _ in W.tensor_specs(cfg)]
    P = {n: torch.from_numpy(np.asarray(t, np.float64)) for n, t in zip(names, tensors)}
    B, S = ids.shape
    hd, nh, kvh = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    cos_t, sin_t = (torch.from_numpy(a.astype(np.float64)) for a in
                    __import__("oracle.orc", fromlist=["x"]).rope_tables(hd, cfg.max_seq, cfg.theta))
    h = P["model.embedTokens.weight"][torch.from_numpy(ids).long()]

    def norm(x, g, b):
        if cfg.norm_kind == 0:
            return g * (x / torch.sqrt((x * x).mean(-1, keepdim=True) + cfg.eps))
        mu = x.mean(-1, keepdim=True)
        c = x - mu
        return g * (c * torch.rsqrt((c * c).mean(-1, keepdim=True) + cfg.eps)) + b

    def rope(x):  # [B,H,S,hd]
        c = cos_t[offset:offset + S, 0::2]
        s = sin_t[offset:offset + S, 0::2]
        x0, x1 = x[..., 0::2], x[..., 1::2]
        return torch.stack([c * x0 - s * x1, s * x0 + c * x1], -1).reshape(x.shape)

    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    vis = (i <= j) if cfg.mask_kind == 0 else (j <= i)
    mask = torch.where(vis, 0.0, -1e9).double()
    for l in range(cfg.n_layers):
        p = "model.layers.%d." % l
        x = norm(h, P[p + "inputLayernorm.gamma"], P[p + "inputLayernorm.beta"])
        q = (x @ P[p + "selfAttn.qProj.weight"] + P[p + "selfAttn.qProj.bias"]).view(B, S, nh, hd).transpose(1, 2)
        k = (x @ P[p + "selfAttn.kProj.weight"] + P[p + "selfAttn.kProj.bias"]).view(B, S, kvh, hd).transpose(1, 2)
        v = (x @ P[p + "selfAttn.vProj.weight"] + P[p + "selfAttn.vProj.bias"]).view(B, S, kvh, hd).transpose(1, 2)
        q, k = rope(q), rope(k)
        k = k.repeat_interleave(nh // kvh, 1)
        v = v.repeat_interleave(nh // kvh, 1)
        sc = q @ k.transpose(-1, -2) * (1.0 / np.sqrt(np.float32(hd)))
        if causal:
            sc = sc + mask
        a = torch.softmax(sc, -1) @ v
        a = a.transpose(1, 2).reshape(B, S, nh * hd)
        h = h + (a @ P[p + "selfAttn.outProj.weight"] + P[p + "selfAttn.outProj.bias"])
        x = norm(h, P[p + "postAttentionLayernorm.gamma"], P[p + "postAttentionLayernorm.beta"])
        g = x @ P[p + "mlp.gateProj.weight"] + P[p + "mlp.gateProj.bias"]
        u = x @ P[p + "mlp.upProj.weight"] + P[p + "mlp.upProj.bias"]
        h = h + ((g * torch.sigmoid(g) * u) @ P[p + "mlp.downProj.weight"] + P[p + "mlp.downProj.bias"])
    h = norm(h, P["model.norm.gamma"], P["model.norm.beta"])
    return (h @ P["lmHead.weight"] + P["lmHead.bias"]).numpy()


@pytest.mark.parametrize("norm_kind,mask_kind", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_oracle_matches_independent_torch_model(orc, norm_kind, mask_kind):
    cfg = W.tiny_llama(norm_kind=norm_kind, mask_kind=mask_kind)
    t = W.init_weights(cfg, seed=11, trivial_affine=False)
    ids = np.random.default_rng(12).integers(0, cfg.vocab, size=(2, 10)).astype(np.int32)
    got = orc.model_forward(cfg, t, ids, offset=3, causal=True)
    want = _torch_forward(cfg, t, ids, 3, True)
    assert rel_l2(got, want) < 2e-6


def test_oracle_f32_accumulation_close_to_f64(orc):
    cfg = W.tiny_llama()
    t = W.init_weights(cfg, seed=0)
    ids = np.random.default_rng(1).integers(0, cfg.vocab, size=(1, 16)).astype(np.int32)
    a = orc.model_forward(cfg, t, ids)
    orc.set_accum64(0)
    try:
        b = orc.model_forward(cfg, t, ids)
    finally:
        orc.set_accum64(1)
    assert rel_l2(b, a) < 1e-5


# ---- committed golden fixtures ---------------------------------------------
def test_golden_tiny_generate_reproduces(orc):
    z = np.load(os.path.join(GOLD, "tiny_llama_generate.npz"))
    cfg = W.tiny_llama(norm_kind=0, mask_kind=0)
    ids, last = orc.generate_greedy(cfg, W.init_weights(cfg, seed=0), z["prompt"], 32)
    assert np.array_equal(ids, z["ids_rms_as_written"])
    assert rel_l2(last, z["last_logits_rms_as_written"]) < 1e-6
    assert np.array_equal(z["prompt"], np.random.default_rng(1).integers(0, 1024, size=(1, 32)).astype(np.int32))


def test_golden_small_ops_reproduce(orc):
    z = np.load(os.path.join(GOLD, "small_ops.npz"))
    np.testing.assert_allclose(orc.linear(z["lin_x"], z["lin_w"], z["lin_b"]), z["lin_y"], rtol=1e-6)
    np.testing.assert_allclose(orc.rmsnorm(z["lin_x"], z["norm_g"]), z["rms_y"], rtol=1e-6)
    np.testing.assert_allclose(orc.gqa_attention(z["att_q"], z["att_k"], z["att_v"], True, 0), z["att_as_written"], rtol=1e-6)
