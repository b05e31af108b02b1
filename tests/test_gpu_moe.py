"""DeepSeek-style MoE on the GPU against the oracle (dense all-experts reference math,
src/rew/models/deepseek.nim:122-145), through the C ABI."""
import os

import numpy as np
import pytest

from conftest import rel_l2
from rew_b200 import weights as W

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def rb():
    from rew_b200 import _lib, api
    _lib.init()
    return api


def test_router_matches_oracle_and_golden(rb, orc):
    z = np.load(os.path.join(GOLD, "small_ops.npz"))
    T = rb.Tensor.from_host
    w, i = rb.moeRoute(T(z["lin_x"]), rb.Linear(T(z["route_w"]), T(z["route_b"])), 3)
    assert np.array_equal(i.to_host(), z["route_topi"])
    np.testing.assert_allclose(w.to_host(), z["route_topw"], rtol=2e-6)
    rng = np.random.default_rng(5)
    x = rng.normal(size=(70, 64)).astype(np.float32)
    rw = rng.normal(0, 0.3, size=(64, 64)).astype(np.float32)
    rbias = rng.normal(0, 0.1, size=(64,)).astype(np.float32)
    w, i = rb.moeRoute(T(x), rb.Linear(T(rw), T(rbias)), 6)
    ow, oi = orc.moe_route(x, rw, rbias, 6)
    assert np.array_equal(i.to_host(), oi)
    np.testing.assert_allclose(w.to_host(), ow, rtol=1e-5)
    np.testing.assert_allclose(w.to_host().sum(-1), 1.0, rtol=1e-6)


def _check_rows(got, want, tol=2e-2, flipped=None):
    """bf16 activations perturb router logits by ~1e-2; where two experts are nearly tied for the k-th
    place the GPU and the f32 oracle can pick different ones, which moves that one token's output by far
    more than the bf16 tolerance (the reference's own topK leaves exact ties unspecified too,
    src/rew/ops/sort.nim:54-59).  So: every sequence within tolerance, except that at most a quarter of
    them (at least one) may sit above it, and none beyond 0.25.  `flipped[b]` says whether the device routed
    some token of sequence b to another SET of experts than the oracle at some layer: a sequence may only be
    out of tolerance if that happened.  The forced-routing test below has no such ambiguity and holds the
    strict bound."""
    per = [rel_l2(got[b], want[b]) for b in range(len(got))]
    over = [b for b, e in enumerate(per) if e > tol]
    assert len(over) <= max(1, len(per) // 4) and max(per) <= 0.25, per
    if flipped is not None:
        for b in over:
            assert flipped[b], "sequence %d is %.3f off the oracle although every router decision agrees" % (b, per[b])


def _flipped_sequences(sess, orc, cfg, t, seq, S_last):
    """Per sequence: did any MoE layer of the device's last forward (the final S_last tokens of `seq`) choose a
    different set of experts for some token than the oracle's forward over `seq`?"""
    B, L = seq.shape
    o_topi, _ = orc.model_routing(cfg, t, seq, 0, True)                 # [n_moe, B, L, k]
    out = np.zeros(B, bool)
    for l in range(o_topi.shape[0]):
        g = sess.routing(l, B * S_last).reshape(B, S_last, -1)
        want = o_topi[l][:, L - S_last:]
        out |= (np.sort(g, -1) != np.sort(want, -1)).any(axis=(1, 2))
    return out


def _moe_cfg(dtype, **kw):
    base = dict(vocab=256, d_model=128, n_layers=3, n_heads=4, n_kv_heads=4, head_dim=32, ffn=192, max_seq=128, theta=10000.0,
                eps=1e-6, n_routed=8, n_shared=2, top_k=3, moe_ffn=64, first_dense=192, dtype=dtype, mask_kind=1)
    base.update(kw)
    return W.ModelConfig(**base)


def test_f32_moe_generate_token_exact(rb, orc):
    from rew_b200 import _lib
    cfg = _moe_cfg(_lib.F32)
    t = W.init_weights(cfg, seed=21, std=0.08, trivial_affine=False)
    prompt = np.random.default_rng(4).integers(0, cfg.vocab, size=(2, 11)).astype(np.int32)
    want_ids, want_logits = orc.generate_greedy(cfg, t, prompt, 6)
    sess = rb.CausalLM(cfg).load(t).session(2, 32)
    ids, logits = sess.generate(prompt, 6, want_logits=True)
    assert np.array_equal(ids, want_ids)
    assert rel_l2(logits, want_logits) <= 1e-5


@pytest.mark.parametrize("n_shared,first_dense", [(2, 192), (0, 0)])
def test_bf16_moe_logits_within_tolerance(rb, orc, n_shared, first_dense):
    from rew_b200 import _lib
    cfg = _moe_cfg(_lib.BF16, head_dim=64, n_heads=2, n_kv_heads=2, n_shared=n_shared, first_dense=first_dense)
    t = W.init_weights(cfg, seed=22, std=0.08, trivial_affine=False)
    # Peaked router: bf16 activations perturb the router logits by ~1e-2, which would flip the k-th
    # choice of near-tied experts against the f32 oracle; with a sharper gate the experts whose order
    # can flip carry negligible weight.
    for i, (name, _) in enumerate(W.tensor_specs(cfg)):
        if name.endswith("moe.gate.weight"):
            t[i] = t[i] * 8.0
    t = [orc.bf16_round(a) if a.ndim == 2 else a for a in t]
    rb.set_option("record_routing", "1")
    try:
        for B, S in ((3, 40), (2, 7)):
            prompt = np.random.default_rng(B).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
            sess = rb.CausalLM(cfg).load(t).session(B, S + 8)
            nxt, logits = sess.forward(prompt, want_logits=True)
            _check_rows(logits, orc.model_forward(cfg, t, prompt, 0, True)[:, -1],
                        flipped=_flipped_sequences(sess, orc, cfg, t, prompt, S))
            ids, last = sess.decode(3, want_logits=True)
            seq = np.concatenate([prompt, nxt[:, None], ids[:, :2]], 1)
            _check_rows(last, orc.model_forward(cfg, t, seq, 0, True)[:, -1])
            sess.free()
    finally:
        rb.set_option("record_routing", "0")


def test_moe_every_token_to_one_expert_is_handled(rb, orc):
    """Ragged extreme: a router bias that sends every token to the same experts (capacity = all pairs)."""
    from rew_b200 import _lib
    cfg = _moe_cfg(_lib.BF16, head_dim=64, n_heads=2, n_kv_heads=2)
    t = [orc.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(cfg, seed=23, std=0.05)]
    names = [n for n, _ in W.tensor_specs(cfg)]
    for l in (1, 2):
        b = np.zeros(8, np.float32)
        b[[1, 4, 6]] = 50.0
        t[names.index("model.layers.%d.moe.gate.bias" % l)] = b
    prompt = np.random.default_rng(9).integers(0, cfg.vocab, size=(4, 33)).astype(np.int32)
    sess = rb.CausalLM(cfg).load(t).session(4, 48)
    nxt, logits = sess.forward(prompt, want_logits=True)
    want = orc.model_forward(cfg, t, prompt, 0, True)[:, -1]
    assert rel_l2(logits, want) <= 2e-2
    ids, last = sess.decode(4, want_logits=True)          # decode steps replay the captured graph
    seq = np.concatenate([prompt, nxt[:, None], ids[:, :3]], 1)
    want = orc.model_forward(cfg, t, seq, 0, True)[:, -1]
    assert rel_l2(last, want) <= 2e-2


def test_moe_local_grouping_matches_slot_path_and_oracle(rb, orc):
    """On one rank, steps of at most 2048 (token, expert) pairs sort the pairs by expert in one kernel;
    larger ones go through the per-peer slot arrays that expert parallelism uses.  An 800-token prompt
    (2400 pairs) fed at once takes the slot path, the same prompt fed in two chunks the sorting kernel:
    both match the oracle, with routing forced by the gate bias so that no near-tie can flip."""
    from rew_b200 import _lib
    cfg = _moe_cfg(_lib.BF16, head_dim=64, n_heads=2, n_kv_heads=2)
    t = [orc.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(cfg, seed=29, std=0.05)]
    names = [n for n, _ in W.tensor_specs(cfg)]
    for l in (1, 2):
        b = np.zeros(8, np.float32)
        b[[0, 3, 7]] = 50.0
        t[names.index("model.layers.%d.moe.gate.bias" % l)] = b
    B, S = 8, 100
    prompt = np.random.default_rng(12).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
    want = orc.model_forward(cfg, t, prompt, 0, True)[:, -1]
    sess = rb.CausalLM(cfg).load(t).session(B, 112)
    _, whole = sess.forward(prompt, want_logits=True)
    sess.reset()
    sess.forward(prompt[:, :50])
    _, chunked = sess.forward(prompt[:, 50:], want_logits=True)
    assert rel_l2(whole, want) <= 2e-2
    assert rel_l2(chunked, want) <= 2e-2
    assert rel_l2(chunked, whole) <= 1e-2
