"""GPU parity of the model engine (prefill, KV-cached decode, generate) with the
CPU oracle and the committed golden fixtures, through the C ABI."""
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


@pytest.mark.parametrize("norm,mask", [("rms", "as_written"), ("rms", "standard"), ("layernorm", "as_written"),
                                       ("layernorm", "standard")])
def test_tiny_llama_fp32_generate_token_exact(rb, norm, mask):
    """The tiny fp32 Llama configuration: greedy ids identical, final logits rel-L2 <= 1e-5."""
    z = np.load(os.path.join(GOLD, "tiny_llama_generate.npz"))
    cfg = W.tiny_llama(norm_kind=0 if norm == "rms" else 1, mask_kind=0 if mask == "as_written" else 1)
    model = rb.CausalLM(cfg).load(W.init_weights(cfg, seed=0))
    sess = model.session(1, 64)
    ids, logits = sess.generate(z["prompt"], 32, eos=-1, want_logits=True)
    assert np.array_equal(ids, z["ids_%s_%s" % (norm, mask)])
    assert rel_l2(logits, z["last_logits_%s_%s" % (norm, mask)]) <= 1e-5
    # a second run through the captured decode graph gives the same ids
    assert np.array_equal(sess.generate(z["prompt"], 32, eos=-1), ids)


def test_tiny_llama_fp32_batched_and_nontrivial_affine(rb, orc):
    cfg = W.tiny_llama(norm_kind=1, mask_kind=1)
    t = W.init_weights(cfg, seed=5, trivial_affine=False)
    prompt = np.random.default_rng(2).integers(0, cfg.vocab, size=(3, 17)).astype(np.int32)
    want_ids, want_last = orc.generate_greedy(cfg, t, prompt, 12)
    sess = rb.CausalLM(cfg).load(t).session(3, 40)
    ids, logits = sess.generate(prompt, 12, want_logits=True)
    assert np.array_equal(ids, want_ids)
    assert rel_l2(logits, want_last) <= 1e-5


@pytest.mark.parametrize("mask_kind", [0, 1])
def test_forward_all_matches_reference_forward(rb, orc, mask_kind):
    """LlamaForCausalLM.forward as written: no cache, logits for every position, RoPE offset."""
    cfg = W.tiny_llama(norm_kind=1, mask_kind=mask_kind)
    t = W.init_weights(cfg, seed=8, trivial_affine=False)
    ids = np.random.default_rng(3).integers(0, cfg.vocab, size=(2, 21)).astype(np.int32)
    sess = rb.CausalLM(cfg).load(t).session(2, 32)
    got = sess.forward_all(ids, offset=4, causal=True)
    assert rel_l2(got, orc.model_forward(cfg, t, ids, 4, True)) <= 1e-5
    got = sess.forward_all(ids, offset=0, causal=False)
    assert rel_l2(got, orc.model_forward(cfg, t, ids, 0, False)) <= 1e-5


def test_generate_stops_at_eos_and_errors(rb, orc):
    from rew_b200._lib import RewB200Error
    z = np.load(os.path.join(GOLD, "tiny_llama_generate.npz"))
    cfg = W.tiny_llama()
    sess = rb.CausalLM(cfg).load(W.init_weights(cfg, seed=0)).session(1, 64)
    gold = z["ids_rms_as_written"][0]
    eos = int(gold[3])
    first = int(np.argmax(gold == eos))
    ids = sess.generate(z["prompt"], 32, eos=eos)[0]
    assert ids[:first + 1].tolist() == gold[:first + 1].tolist()
    assert (ids[first + 1:] == -1).all()
    with pytest.raises(RewB200Error, match="exceeds maxLen"):
        sess.generate(z["prompt"], 40)
    with pytest.raises(RewB200Error, match="token id out of range"):
        sess.forward(np.array([[cfg.vocab]], np.int32))
    with pytest.raises(RewB200Error, match="divisible by numKVHeads"):
        rb.CausalLM(W.ModelConfig(vocab=32, d_model=24, n_layers=1, n_heads=3, n_kv_heads=2, head_dim=8, ffn=16))


def _small_bf16_cfg(**kw):
    from rew_b200 import _lib
    return W.ModelConfig(vocab=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64, ffn=688, max_seq=256,
                         theta=500000.0, dtype=_lib.BF16, mask_kind=1, **kw)


@pytest.mark.parametrize("B,S", [(1, 5), (3, 70), (32, 16), (2, 130)])
def test_bf16_model_logits_within_tolerance(rb, orc, B, S):
    """bf16 weights and activations against f32 oracle math on the bf16-rounded weights: rel-L2 <= 2e-2."""
    cfg = _small_bf16_cfg()
    t = [orc.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(cfg, seed=4, std=0.05, trivial_affine=False)]
    prompt = np.random.default_rng(B).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
    sess = rb.CausalLM(cfg).load(t).session(B, S + 8)
    nxt, logits = sess.forward(prompt, want_logits=True)
    want = orc.model_forward(cfg, t, prompt, 0, True)[:, -1]
    assert rel_l2(logits, want) <= 2e-2
    # teacher-forced decode step: feed the oracle's greedy token, compare the next logits
    ids, last = sess.decode(3, want_logits=True)
    seq = np.concatenate([prompt, nxt[:, None], ids[:, :2]], 1)
    want = orc.model_forward(cfg, t, seq, 0, True)[:, -1]
    assert rel_l2(last, want) <= 2e-2


@pytest.mark.parametrize("B,S,n", [(4, 100, 9), (48, 40, 3), (100, 24, 3), (200, 12, 3)])
def test_bf16_cached_decode_equals_prefill_recompute(rb, B, S, n):
    """Size-independent property at a wider config: logits after n cached decode steps equal the
    logits of one prefill over the same tokens (same kernels' math, different schedule).  The batch
    sizes cover the decode tiles of 32, 64, 128 and 256 rows, each with its own split-K depth."""
    from rew_b200 import _lib
    cfg = W.ModelConfig(vocab=2048, d_model=1024, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=128, ffn=2816, max_seq=512,
                        theta=500000.0, dtype=_lib.BF16, mask_kind=1)
    model = rb.CausalLM(cfg).init_random(seed=1, std=0.02)
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
    sess = model.session(B, 256)
    first = sess.forward(prompt)
    ids, last = sess.decode(n, want_logits=True)
    seq = np.concatenate([prompt, first[:, None], ids[:, :n - 1]], 1)
    sess.reset()
    _, again = sess.forward(seq, want_logits=True)
    assert rel_l2(last, again) <= 2e-2
    assert np.isfinite(last).all()


def test_launch_counter_moves(rb):
    from rew_b200 import _lib
    before = _lib.lib().rewb200_launch_count(0)
    cfg = W.tiny_llama()
    sess = rb.CausalLM(cfg).load(W.init_weights(cfg, seed=0)).session(1, 16)
    sess.forward(np.array([[1, 2, 3]], np.int32))
    assert _lib.lib().rewb200_launch_count(0) > before


def test_bf16_prefill_attention_kernels_agree_and_chunked_prefill(rb):
    """head_dim 128 and prompts of 128+ tokens put prefill attention on the tcgen05 kernel: its logits match
    the mma.sync kernel's, and a prompt fed in two chunks (the second attends to a 150-token context through
    the paged cache) matches the same prompt fed at once."""
    from rew_b200 import _lib
    cfg = W.ModelConfig(vocab=1024, d_model=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, max_seq=512,
                        theta=500000.0, dtype=_lib.BF16, mask_kind=1)
    model = rb.CausalLM(cfg).init_random(seed=2, std=0.04)
    B, S = 3, 300
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
    sess = model.session(B, 320)
    _, a = sess.forward(prompt, want_logits=True)
    rb.set_option("attention", "mma")
    try:
        sess.reset()
        _, b = sess.forward(prompt, want_logits=True)
    finally:
        rb.set_option("attention", "tc")
    assert np.isfinite(a).all() and rel_l2(a, b) <= 1e-2
    sess.reset()
    sess.forward(prompt[:, :150])
    _, c = sess.forward(prompt[:, 150:], want_logits=True)
    assert rel_l2(c, a) <= 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("norm_kind,d_model", [(0, 512), (1, 512), (0, 2064)])
def test_bf16_decode_norm_kernels_agree(rb, norm_kind, d_model):
    """Decode-size residual+norm runs on clusters of four CTAs per row (row statistics exchanged through
    distributed shared memory); option norm=row keeps one CTA per row.  Both compute the same rmsNorm /
    LayerNorm of the same f32 residual stream, so the bf16 logits of a prompt plus a few decode steps
    agree to summation-order rounding."""
    from rew_b200 import _lib
    cfg = W.ModelConfig(vocab=512, d_model=d_model, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64, ffn=768, max_seq=64,
                        theta=10000.0, dtype=_lib.BF16, norm_kind=norm_kind)
    model = rb.CausalLM(cfg).init_random(seed=5, std=0.05)
    B = 5
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, size=(B, 7)).astype(np.int32)
    outs = {}
    for mode in ("cluster", "row"):
        rb.set_option("norm", mode)
        try:
            sess = model.session(B, 32)
            _, first = sess.forward(prompt, want_logits=True)
            _, last = sess.decode(6, want_logits=True)
            outs[mode] = (first, last)
        finally:
            rb.set_option("norm", "cluster")
    a, b = outs["cluster"], outs["row"]
    assert np.isfinite(a[0]).all() and rel_l2(a[0], b[0]) <= 2e-3
    assert np.isfinite(a[1]).all() and rel_l2(a[1], b[1]) <= 5e-3


@pytest.mark.gpu
@pytest.mark.parametrize("head_dim,n_heads,n_kv", [(128, 8, 2), (64, 6, 3)])
def test_bf16_decode_cluster_splitk_matches_slabs_and_oracle(rb, orc, head_dim, n_heads, n_kv):
    """With option splitk=cluster, steps of at most 32 rows sum their split-K slices inside thread-block
    clusters and the q|k|v launch finishes bias, RoPE and the cache write in its epilogue; splitk=slabs
    (the default) leaves f32 slabs for the next kernel.  Same sums in the same order: the logits of a
    21-row prompt (3 sequences x 7 tokens) and of decode steps agree to bf16 rounding of q/k, and both
    stay within the bf16 tolerance of the oracle."""
    from rew_b200 import _lib
    cfg = W.ModelConfig(vocab=512, d_model=1024, n_layers=2, n_heads=n_heads, n_kv_heads=n_kv, head_dim=head_dim, ffn=2048,
                        max_seq=128, theta=10000.0, dtype=_lib.BF16, mask_kind=1)
    t = [orc.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(cfg, seed=9, std=0.03, trivial_affine=False)]
    B, S = 3, 7
    prompt = np.random.default_rng(4).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
    outs = {}
    for mode in ("cluster", "slabs"):
        rb.set_option("splitk", mode)
        try:
            sess = rb.CausalLM(cfg).load(t).session(B, 64)
            nxt, first = sess.forward(prompt, want_logits=True)
            ids, last = sess.decode(4, want_logits=True)
            outs[mode] = (nxt, first, ids, last)
        finally:
            rb.set_option("splitk", "slabs")
    a, b = outs["cluster"], outs["slabs"]
    assert np.isfinite(a[1]).all() and np.isfinite(a[3]).all()
    assert rel_l2(a[1], b[1]) <= 2e-3
    want = orc.model_forward(cfg, t, prompt, 0, True)[:, -1]
    assert rel_l2(a[1], want) <= 2e-2
    if np.array_equal(a[0], b[0]) and np.array_equal(a[2], b[2]):
        assert rel_l2(a[3], b[3]) <= 5e-3
    seq = np.concatenate([prompt, a[0][:, None], a[2][:, :3]], 1)
    want = orc.model_forward(cfg, t, seq, 0, True)[:, -1]
    assert rel_l2(a[3], want) <= 2e-2


@pytest.mark.gpu
def test_model_from_hf_snapshot_directory(rb, orc, tmp_path):
    """config.json + sharded safetensors with Hugging Face names -> model on the device; greedy ids equal the
    oracle's on the converted weights (fp32, token-exact)."""
    import json
    from rew_b200 import safetensors as ST
    cfg = W.tiny_llama(mask_kind=1, norm_kind=0)
    rng = np.random.default_rng(3)
    d, hd = cfg.d_model, cfg.head_dim
    hf = {"model.embed_tokens.weight": rng.normal(0, 0.05, (cfg.vocab, d)), "model.norm.weight": 1 + 0.1 * rng.normal(size=d),
          "lm_head.weight": rng.normal(0, 0.05, (cfg.vocab, d))}
    for l in range(cfg.n_layers):
        p = "model.layers.%d." % l
        hf[p + "self_attn.q_proj.weight"] = rng.normal(0, 0.05, (cfg.n_heads * hd, d))
        hf[p + "self_attn.k_proj.weight"] = rng.normal(0, 0.05, (cfg.n_kv_heads * hd, d))
        hf[p + "self_attn.v_proj.weight"] = rng.normal(0, 0.05, (cfg.n_kv_heads * hd, d))
        hf[p + "self_attn.o_proj.weight"] = rng.normal(0, 0.05, (d, cfg.n_heads * hd))
        hf[p + "mlp.gate_proj.weight"] = rng.normal(0, 0.05, (cfg.ffn, d))
        hf[p + "mlp.up_proj.weight"] = rng.normal(0, 0.05, (cfg.ffn, d))
        hf[p + "mlp.down_proj.weight"] = rng.normal(0, 0.05, (d, cfg.ffn))
        hf[p + "input_layernorm.weight"] = 1 + 0.1 * rng.normal(size=d)
        hf[p + "post_attention_layernorm.weight"] = 1 + 0.1 * rng.normal(size=d)
    hf = {k: v.astype(np.float32) for k, v in hf.items()}
    names = sorted(hf)
    half = len(names) // 2
    ST.write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), {k: hf[k] for k in names[:half]})
    ST.write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), {k: hf[k] for k in names[half:]})
    (tmp_path / "config.json").write_text(json.dumps({
        "vocab_size": cfg.vocab, "hidden_size": cfg.d_model, "intermediate_size": cfg.ffn, "num_hidden_layers": cfg.n_layers,
        "num_attention_heads": cfg.n_heads, "num_key_value_heads": cfg.n_kv_heads, "max_position_embeddings": cfg.max_seq,
        "rope_theta": cfg.theta, "rms_norm_eps": cfg.eps}))
    model = rb.CausalLM.from_hf_snapshot(str(tmp_path))
    prompt = np.random.default_rng(5).integers(0, cfg.vocab, size=(2, 9)).astype(np.int32)
    got = model.session(2, 32).generate(prompt, 8)
    loaded = ST.llama_from_hf(model.cfg, ST.read_safetensors_dir(str(tmp_path)))
    want, _ = orc.generate_greedy(model.cfg, loaded, prompt, 8)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("nth", [1, 3, 6])
def test_failed_activation_growth_leaves_the_session_usable(rb, orc, nth):
    """An allocation that fails while the activation buffers grow (injected on the host, the device is not
    touched) is reported as an error, and the session then allocates again on the next call instead of
    launching kernels on freed or NULL buffers."""
    from rew_b200 import _lib
    cfg = W.tiny_llama(mask_kind=1)
    t = W.init_weights(cfg, seed=0)
    prompt = np.random.default_rng(7).integers(0, cfg.vocab, size=(1, 12)).astype(np.int32)
    want_ids, _ = orc.generate_greedy(cfg, t, prompt, 5)
    sess = rb.CausalLM(cfg).load(t).session(1, 48)
    assert np.array_equal(sess.generate(prompt[:, :4], 2).shape, (1, 2))      # buffers sized for 4 rows exist now
    rb.set_option("inject_alloc_fail", str(nth))
    try:
        with pytest.raises(_lib.RewB200Error, match="injected"):
            sess.generate(prompt, 5)                                              # 12 rows: growth fails part-way
    finally:
        rb.set_option("inject_alloc_fail", "0")
    assert np.array_equal(sess.generate(prompt[:, :4], 2).shape, (1, 2))      # fewer rows than the old capacity
    assert np.array_equal(sess.generate(prompt, 5), want_ids)


def test_l8_shaped_layer_bf16_batch32_against_oracle(rb, orc):
    """One decoder layer with Llama-3-8B's shapes (d_model 4096, 32 query / 8 kv heads, head_dim 128, SwiGLU
    14336; the vocabulary cut to 32064 to keep the host arrays small) plus lm_head, bf16, batch 32: the shapes
    the benchmark's decode step runs (32-row tcgen05 Linear tiles with split-K, cluster norm, split-KV decode
    attention), against f32 oracle math on the bf16-rounded weights.  Prefill of 4 tokens per sequence, then two
    cached decode steps."""
    from rew_b200 import _lib
    cfg = W.llama3_8b()
    cfg.n_layers, cfg.vocab, cfg.max_seq = 1, 32064, 64
    rng = np.random.default_rng(3)
    t = []
    for name, shape in W.tensor_specs(cfg):   # N(0, 0.02) matrices rounded to bf16, zero biases, unit gammas
        if len(shape) == 2:
            a = rng.standard_normal(size=shape, dtype=np.float32)
            a *= 0.02
            t.append(orc.bf16_round(a))
        else:
            t.append(np.ones(shape, np.float32) if name.endswith("gamma") else np.zeros(shape, np.float32))
    B, S = 32, 4
    prompt = np.random.default_rng(8).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
    sess = rb.CausalLM(cfg).load(t).session(B, 16)
    nxt, logits = sess.forward(prompt, want_logits=True)
    want = orc.model_forward(cfg, t, prompt, 0, True)[:, -1]
    assert rel_l2(logits, want) <= 2e-2
    assert max(rel_l2(logits[b], want[b]) for b in range(B)) <= 2e-2
    ids, last = sess.decode(2, want_logits=True)
    seq = np.concatenate([prompt, nxt[:, None], ids[:, :1]], 1)
    want = orc.model_forward(cfg, t, seq, 0, True)[:, -1]
    assert rel_l2(last, want) <= 2e-2
    assert max(rel_l2(last[b], want[b]) for b in range(B)) <= 2e-2


def test_qkv_finish_inside_attention_equals_the_separate_launch(rb):
    """Decode steps finish q / k / v of the new token (slab sum, bias, RoPE, cache append) inside the attention kernel
    by default; option qkv_post=launch runs the separate kernel of the prefill path instead.  Same arithmetic in
    the same order: identical ids and logits, with split-KV (long context, one sequence) and without."""
    from rew_b200 import _lib
    cfg = W.ModelConfig(vocab=512, d_model=512, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=128, ffn=1024, max_seq=1024,
                        theta=500000.0, dtype=_lib.BF16, mask_kind=1)
    t = [W.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(cfg, seed=6, std=0.05, trivial_affine=False)]
    model = rb.CausalLM(cfg).load(t)
    # 160 sequences x 2 kv heads = 320 CTAs: more than one wave, where the default keeps the separate launch and only
    # attention_always fuses
    for B, S in ((1, 700), (5, 63), (3, 64), (160, 9)):
        prompt = np.random.default_rng(B + S).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
        outs = []
        for how in ("attention_always", "launch"):
            rb.set_option("qkv_post", how)
            try:
                sess = model.session(B, S + 16)
                outs.append(sess.generate(prompt, 9, want_logits=True))
                sess.free()
            finally:
                rb.set_option("qkv_post", "attention")
        assert np.array_equal(outs[0][0], outs[1][0])
        assert np.array_equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("key,other,default", [("gate_up_split", "off", "on"), ("splitk_min_blocks", "2", "8")])
def test_decode_splitk_policy_switches_agree(rb, orc, key, other, default):
    """gate_up_split=off keeps a narrow gate|up launch in one piece (SwiGLU in the GEMM epilogue) instead of
    K slices + a sum-and-SwiGLU launch; splitk_min_blocks lets a K slice get shorter.  Both change only the order
    in which f32 partial sums are added, so logits agree far inside the bf16 tolerance, and both settings stay
    within it against the oracle."""
    from rew_b200 import _lib
    cfg = W.ModelConfig(vocab=512, d_model=2048, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, max_seq=128,
                        theta=500000.0, dtype=_lib.BF16, mask_kind=1)
    t = [orc.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(cfg, seed=13, std=0.03, trivial_affine=False)]
    B, S = 4, 9
    prompt = np.random.default_rng(14).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
    outs = {}
    for val in (default, other):
        rb.set_option(key, val)
        try:
            sess = rb.CausalLM(cfg).load(t).session(B, 64)
            nxt, _ = sess.forward(prompt, want_logits=True)
            ids, last = sess.decode(3, want_logits=True)
            outs[val] = (nxt, ids, last)
        finally:
            rb.set_option(key, default)
    a, b = outs[default], outs[other]
    if np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]):
        assert rel_l2(a[2], b[2]) <= 5e-3
    for nxt, ids, last in (a, b):
        seq = np.concatenate([prompt, nxt[:, None], ids[:, :2]], 1)
        want = orc.model_forward(cfg, t, seq, 0, True)[:, -1]
        assert rel_l2(last, want) <= 2e-2
