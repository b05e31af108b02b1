"""The stateful layer entry points of the C ABI against the oracle: GroupedQueryAttention with an in-place
KvCache (src/rew/nn/groupedqueryattention.nim:94-144, src/rew/nn/kv_cache.nim:47-77), the routed experts of
DeepSeekMoE.forward (src/rew/models/deepseek.nim:140-144), lm_head + sampling
(src/rew/infer/generate.nim:92-190) and generate's stopTokenIds (generate.nim:263)."""
import numpy as np
import pytest

from conftest import rel_l2
from rew_b200 import weights as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rb():
    from rew_b200 import _lib, api
    _lib.init()
    return api


def _gqa_oracle(orc, x, w, nh, kvh, hd, theta, max_seq):
    """No-cache recompute of the whole sequence with the conventional causal mask."""
    B, L, d = x.shape
    q = orc.linear(x.reshape(B * L, d), w["q"], w["qb"]).reshape(B, L, nh, hd).transpose(0, 2, 1, 3)
    k = orc.linear(x.reshape(B * L, d), w["k"], w["kb"]).reshape(B, L, kvh, hd).transpose(0, 2, 1, 3)
    v = orc.linear(x.reshape(B * L, d), w["v"], w["vb"]).reshape(B, L, kvh, hd).transpose(0, 2, 1, 3)
    c, s = orc.rope_tables(hd, max_seq, theta)
    q, k = orc.rope_apply(np.ascontiguousarray(q), c, s, 0), orc.rope_apply(np.ascontiguousarray(k), c, s, 0)
    a = orc.gqa_attention(q, k, np.ascontiguousarray(v), True, 1)
    a = a.transpose(0, 2, 1, 3).reshape(B * L, nh * hd)
    return orc.linear(a, w["o"], w["ob"]).reshape(B, L, d)


@pytest.mark.parametrize("dtype_name,nh,kvh,hd,tol", [("f32", 4, 2, 32, 1e-5), ("bf16", 4, 2, 64, 2e-2), ("bf16", 8, 2, 128, 2e-2)])
def test_gqa_with_cache_equals_recompute(rb, orc, dtype_name, nh, kvh, hd, tol):
    """Prefill of 70 tokens, then three single-token steps through the cache, equal the oracle's no-cache
    recompute of all 73 positions (decode-with-cache == recompute under the conventional mask)."""
    from rew_b200 import _lib
    dt = _lib.F32 if dtype_name == "f32" else _lib.BF16
    rnd = (lambda a: a) if dt == _lib.F32 else orc.bf16_round
    rng = np.random.default_rng(hd)
    B, S, steps, d, max_seq = 2, 70, 3, 128, 96
    x = rnd(rng.normal(size=(B, S + steps, d)).astype(np.float32))
    w = {"q": rnd(rng.normal(0, 0.08, (d, nh * hd)).astype(np.float32)), "k": rnd(rng.normal(0, 0.08, (d, kvh * hd)).astype(np.float32)),
         "v": rnd(rng.normal(0, 0.08, (d, kvh * hd)).astype(np.float32)), "o": rnd(rng.normal(0, 0.08, (nh * hd, d)).astype(np.float32)),
         "qb": rng.normal(0, 0.05, nh * hd).astype(np.float32), "kb": rng.normal(0, 0.05, kvh * hd).astype(np.float32),
         "vb": rng.normal(0, 0.05, kvh * hd).astype(np.float32), "ob": rng.normal(0, 0.05, d).astype(np.float32)}
    want = _gqa_oracle(orc, x, w, nh, kvh, hd, 10000.0, max_seq)
    T = rb.Tensor.from_host
    lin = lambda wk, bk: rb.Linear(T(w[wk], dt), T(w[bk]))
    attn = rb.GroupedQueryAttention(lin("q", "qb"), lin("k", "kb"), lin("v", "vb"), lin("o", "ob"),
                                    rb.RotaryPositionEncoding(hd, max_seq, 10000.0), mask_kind=1)
    cache = rb.KvCache(B, kvh, hd, max_seq, dt)
    got = [attn.forward(T(x[:, :S], dt), cache).to_host()]
    assert cache.length == S
    for t in range(steps):
        got.append(attn.forward(T(x[:, S + t:S + t + 1], dt), cache).to_host())
    assert cache.length == S + steps
    got = np.concatenate(got, 1)
    assert rel_l2(got[:, :S], want[:, :S]) <= tol
    for t in range(steps):
        assert rel_l2(got[:, S + t], want[:, S + t]) <= tol
    with pytest.raises(_lib.RewB200Error, match="exceeds maxLen"):
        attn.forward(T(x[:, :30], dt), cache)
    cache.reset()
    assert cache.length == 0
    again = attn.forward(T(x[:, :S], dt), cache).to_host()
    assert np.array_equal(again, got[:, :S])


def _experts_oracle(orc, x, topw, topi, ex):
    y = np.zeros_like(x, dtype=np.float64)
    for e, (gw, gb, uw, ub, dw, db) in enumerate(ex):
        sel = (topi == e)
        wt = (topw * sel).sum(-1)
        rows = np.nonzero(wt)[0]
        if rows.size:
            y[rows] += wt[rows, None].astype(np.float64) * orc.gated_ffn(x[rows], gw, gb, uw, ub, dw, db)
    return y.astype(np.float32)


@pytest.mark.parametrize("dtype_name,T,d,f,E,k,tol", [
    ("f32", 40, 64, 48, 8, 3, 1e-5),
    ("bf16", 70, 128, 64, 8, 3, 2e-2),      # 210 pairs: sorted in one kernel; 70 > 64 rows per group bound: tcgen05 grouped GEMM
    ("bf16", 24, 128, 64, 8, 2, 2e-2),      # small groups: the weight-streaming mma.sync kernel
    ("bf16", 1200, 256, 192, 16, 4, 2e-2),  # 4800 pairs through the slot arrays, several 256-token tiles, ragged groups
])
def test_routed_experts_match_oracle(rb, orc, dtype_name, T, d, f, E, k, tol):
    from rew_b200 import _lib
    dt = _lib.F32 if dtype_name == "f32" else _lib.BF16
    rnd = (lambda a: a) if dt == _lib.F32 else orc.bf16_round
    rng = np.random.default_rng(T + E)
    x = rnd(rng.normal(size=(T, d)).astype(np.float32))
    rw = rng.normal(0, 0.5, (d, E)).astype(np.float32)
    if E == 16:
        rw[:, 5] = 0  # an expert that (almost) nobody picks, and a crowded one
        rw[:, 2] *= 3
    topw, topi = orc.moe_route(x, rw, np.zeros(E, np.float32), k)
    ex = []
    for e in range(E):
        ex.append((rnd(rng.normal(0, 0.1, (d, f)).astype(np.float32)), rng.normal(0, 0.05, f).astype(np.float32),
                   rnd(rng.normal(0, 0.1, (d, f)).astype(np.float32)), rng.normal(0, 0.05, f).astype(np.float32),
                   rnd(rng.normal(0, 0.1, (f, d)).astype(np.float32)), rng.normal(0, 0.05, d).astype(np.float32)))
    want = _experts_oracle(orc, x, topw, topi, ex)
    Tn = rb.Tensor.from_host
    experts = rb.RoutedExperts([(rb.Linear(Tn(gw, dt), Tn(gb)), rb.Linear(Tn(uw, dt), Tn(ub)), rb.Linear(Tn(dw, dt), Tn(db)))
                                for gw, gb, uw, ub, dw, db in ex])
    got = experts.forward(Tn(x, dt), Tn(topw), Tn(topi.astype(np.int32))).to_host()
    assert got.shape == (T, d)
    assert rel_l2(got, want) <= tol
    per_row = np.linalg.norm(got - want, axis=1) / np.maximum(np.linalg.norm(want, axis=1), 1e-6)
    assert per_row.max() <= 10 * tol  # no single token far off (a mis-routed row would be)
    experts.free()


def test_lmhead_greedy_and_sampled_match_oracle(rb, orc):
    rng = np.random.default_rng(8)
    B, d, V = 5, 64, 3000
    x = rng.normal(size=(B, d)).astype(np.float32)
    w = rng.normal(0, 0.3, (d, V)).astype(np.float32)
    b = rng.normal(0, 0.1, V).astype(np.float32)
    logits = orc.linear(x, w, b)
    T = rb.Tensor.from_host
    head = rb.Linear(T(w), T(b))
    ids, got = rb.lmHeadSample(T(x), head, want_logits=True)
    assert rel_l2(got, logits) <= 1e-5
    assert np.array_equal(ids, logits.argmax(-1).astype(np.int32))          # sampleGreedy: first maximum
    seeds = np.arange(11, 11 + B, dtype=np.uint64)
    for kind, kw in (("k", dict(top_k=40, top_p=1.0)), ("p", dict(top_k=0, top_p=0.8))):
        smp = rb.Sampler(B, V, 16, temperature=1.0, seeds=seeds, **kw)
        ids, got = rb.lmHeadSample(T(x), head, smp, want_logits=True)
        for r in range(B):  # step 0 of generate: key = initKey(seed), logits untouched at temperature 1
            want = orc.sample_top_k(got[r], 40, int(seeds[r])) if kind == "k" else orc.sample_top_p(got[r], 0.8, int(seeds[r]))
            assert ids[r] == want, (kind, r)
        smp.free()


def test_generate_stops_at_stop_token_ids(rb, orc):
    from rew_b200 import _lib
    cfg = W.tiny_llama()
    t = W.init_weights(cfg, seed=0)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, size=(2, 12)).astype(np.int32)
    free_ids, _ = orc.generate_greedy(cfg, t, prompt, 12)
    stop_a, stop_b = int(free_ids[0, 3]), int(free_ids[1, 6])
    sess = rb.CausalLM(cfg).load(t).session(2, 32)
    got = sess.generate(prompt, 12, stop_ids=[stop_a, stop_b])
    for r in range(2):
        hits = [i for i, v in enumerate(free_ids[r]) if int(v) in (stop_a, stop_b)]
        end = hits[0]
        assert np.array_equal(got[r, :end + 1], free_ids[r, :end + 1])       # the stop token itself is part of the output
        assert (got[r, end + 1:] == -1).all()
    # eos and stopTokenIds combine (generate.nim:263)
    got2 = sess.generate(prompt, 12, eos=stop_a, stop_ids=[stop_b])
    assert np.array_equal(got, got2)
