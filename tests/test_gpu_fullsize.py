"""Properties that hold at the benchmark's full model sizes, where the CPU oracle is too slow to be the checker:
with random weights of the Llama-3-8B shape (config 3) and of the DeepSeek-V2-Lite shape (config 5) a sequence's
tokens and logits must not depend on where in the batch it sits, nor on who its neighbours are.  Every row of a
step is an independent row of every GEMM, attention and routing are per sequence, and a token adds its experts'
results in fixed order, so the results are equal bit for bit."""
import numpy as np
import pytest

from rew_b200 import weights as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rb():
    from rew_b200 import _lib, api
    _lib.init()
    return api


def _run(model, prompt, steps):
    sess = model.session(prompt.shape[0], prompt.shape[1] + steps + 8)
    ids, logits = sess.generate(prompt, steps, want_logits=True)
    sess.free()
    return ids, logits


@pytest.mark.parametrize("shape", ["llama3_8b", "deepseek_v2_lite", "llama3_8b_nf4", "llama3_8b_as_written"])
def test_full_size_decode_is_independent_of_batch_position(rb, shape):
    cfg = getattr(W, shape.replace("_nf4", "").replace("_as_written", ""))()
    if shape.endswith("_nf4"):
        cfg.weight_quant = 1      # NF4 block weights: the quantised GEMV for the decode steps, expanded codes for the prefill
    if shape.endswith("_as_written"):
        cfg.mask_kind, cfg.norm_kind = 0, 1   # the reference as written: makeCausalMask's direction, LayerNorm in the layers
    B, S, steps = (64, 48, 6) if shape == "deepseek_v2_lite" else (32, 96, 6)
    cfg.max_seq = 256
    model = rb.CausalLM(cfg).init_random(seed=21, std=0.02)
    try:
        rng = np.random.default_rng(5)
        prompt = rng.integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
        ids, logits = _run(model, prompt, steps)
        assert np.isfinite(logits).all()
        assert (ids >= 0).all() and (ids < cfg.vocab).all()
        perm = rng.permutation(B)
        ids_p, logits_p = _run(model, prompt[perm], steps)
        assert np.array_equal(ids_p, ids[perm])
        assert np.array_equal(logits_p, logits[perm])
        # a sequence among other neighbours (half of the batch replaced): the kept rows do not move
        other = prompt.copy()
        other[B // 2:] = rng.integers(0, cfg.vocab, size=(B - B // 2, S)).astype(np.int32)
        ids_o, logits_o = _run(model, other, steps)
        assert np.array_equal(ids_o[:B // 2], ids[:B // 2])
        assert np.array_equal(logits_o[:B // 2], logits[:B // 2])
    finally:
        model.free()


def _rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def test_full_size_cached_decode_matches_the_uncached_forward(rb):
    """Llama-3-8B shape: the logits of a cached decode step (32-row GEMV tiles, split-K slabs, split-KV decode
    attention, q / k / v finished inside it) against the logits the cache-free forward gives for the same tokens
    (prefill tiles, prefill attention): two different sets of kernels for the same arithmetic.  Both round to bf16
    at the same places but add in different orders, and the difference between them grows with the square root of
    the depth (measured: 0.006 at one layer, 0.012 at 4, 0.024 at 16, 0.033 at 32 with these random weights), so
    the bound here is 5e-2 at 32 layers; the 2e-2 bound against f32 oracle math is held per layer at this width
    in tests/test_gpu_model.py.  The greedy tokens agree up to near-ties of the flat random-weight logits."""
    cfg = W.llama3_8b()
    cfg.max_seq = 256
    model = rb.CausalLM(cfg).init_random(seed=22, std=0.02)
    try:
        B, S, steps = 8, 130, 4
        prompt = np.random.default_rng(6).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
        sess = model.session(B, S + steps + 8)
        ids, last = sess.generate(prompt, steps, want_logits=True)
        seq = np.concatenate([prompt, ids[:, :steps - 1]], 1)
        full = sess.forward_all(seq)            # [B, S + steps - 1, vocab]
        sess.free()
        want = full[:, -1]
        assert max(_rel_l2(last[b], want[b]) for b in range(B)) <= 5e-2
        # the cache-free forward picks the same greedy tokens at the positions the decode steps produced
        # (random weights give flat logits: near-ties may flip, but not more than three of the 32 tokens)
        greedy = full[:, S - 1:, :].argmax(-1)  # predictions for positions S .. S + steps - 1
        assert (greedy != ids).sum() <= 3
        # the prefill of the session and the cache-free forward run the same kernels on the prompt: equal
        sess2 = model.session(B, S + 8)
        _, pre = sess2.forward(prompt, want_logits=True)
        sess2.free()
        assert np.array_equal(pre, full[:, S - 1])
    finally:
        model.free()


def test_full_size_long_context_alone_and_in_a_batch(rb):
    """Llama-3-8B shape, 1500-token prompts: a sequence decoded alone (16 KV splits) and the same sequence inside a
    batch of four (9 splits) see the same prefill (bit-equal logits) but different split-KV partitions in the
    decode steps.  A split rounds its probabilities to bf16 relative to its own running maximum, so two partitions
    differ by bf16 rounding noise in every attention output: 4e-3 rel-L2 in the logits of a one-layer model, growing
    with the square root of the depth to 2.5e-2 at 32 layers (measured); bound 5e-2, same tokens up to one near-tie."""
    cfg = W.llama3_8b()
    cfg.max_seq = 2048
    model = rb.CausalLM(cfg).init_random(seed=23, std=0.02)
    try:
        B, S, steps = 4, 1500, 4
        prompt = np.random.default_rng(7).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
        ids, logits = _run(model, prompt, steps)
        assert np.isfinite(logits).all()
        ids1, logits1 = _run(model, prompt[2:3], steps)
        assert _rel_l2(logits1[0], logits[2]) <= 5e-2
        assert (ids1[0] != ids[2]).sum() <= 1
        sess = model.session(B, S + 8)
        _, pre = sess.forward(prompt, want_logits=True)
        sess.free()
        sess = model.session(1, S + 8)
        _, pre1 = sess.forward(prompt[2:3], want_logits=True)
        sess.free()
        assert np.array_equal(pre1[0], pre[2])      # 1500 rows alone, 6000 rows in the batch: the same bits
    finally:
        model.free()


def test_full_size_moe_prefill_grouped_gemm_kernels_agree(rb):
    """DeepSeek-V2-Lite shape, 64 sequences x 128 tokens (768 rows per expert on average): the prefill's expert GEMMs on
    the persistent tcgen05 kernel with its device-built tile list against the same forward with every Linear on the
    mma.sync kernels (option linear=mma).  Same routing (the router runs ahead of the experts on identical inputs in
    the first MoE layer; later a near-tie may route a token differently, which moves that one sequence), so the
    median sequence agrees to bf16 summation-order noise and at most a few sequences differ more."""
    cfg = W.deepseek_v2_lite()
    cfg.max_seq = 256
    model = rb.CausalLM(cfg).init_random(seed=24, std=0.02)
    try:
        B, S = 64, 128
        prompt = np.random.default_rng(8).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
        outs = {}
        for impl in ("tc", "mma"):
            rb.set_option("linear", impl)
            try:
                sess = model.session(B, S + 8)
                outs[impl] = sess.forward(prompt, want_logits=True)[1]
                sess.free()
            finally:
                rb.set_option("linear", "tc")
        assert np.isfinite(outs["tc"]).all()
        r = np.array([_rel_l2(outs["tc"][b], outs["mma"][b]) for b in range(B)])
        assert np.median(r) <= 2e-2
        assert (r > 5e-2).sum() <= B // 8
    finally:
        model.free()


def test_full_size_prefill_kernel_variants_return_the_same_bits(rb):
    """Llama-3-8B shape, 8 x 512-token prompts: the prefill with the two-CTA Linear (default), the one-CTA persistent
    Linear and the one-tile Linear, and with one or two query tiles per CTA in the attention kernel.  All variants
    issue the same products in the same order and share their epilogue and softmax arithmetic: identical logits."""
    cfg = W.llama3_8b()
    cfg.max_seq = 640
    model = rb.CausalLM(cfg).init_random(seed=25, std=0.02)
    try:
        B, S = 8, 512
        prompt = np.random.default_rng(9).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)

        def run(**opts):
            for k, v in opts.items():
                rb.set_option(k, v)
            try:
                sess = model.session(B, S + 8)
                out = sess.forward(prompt, want_logits=True)[1]
                sess.free()
                return out
            finally:
                rb.set_option("prefill", "pair")
                rb.set_option("attention", "tc")

        base = run()
        assert np.isfinite(base).all()
        for opts in ({"prefill": "persistent"}, {"prefill": "tile"}, {"attention": "tc2"}, {"attention": "tc1"}):
            assert np.array_equal(run(**opts), base), opts
    finally:
        model.free()


def test_full_size_decode_launch_variants_return_the_same_bits(rb):
    """Llama-3-8B shape, 4 x 1200-token prompts (9 KV splits per sequence and kv head) and 32 x 100-token prompts (no
    split): decode steps with q / k / v finished inside the attention kernel or in a launch of their own, and with the
    split-KV partials merged by a launch or by the last CTA of a sequence.  Same arithmetic in the same order."""
    cfg = W.llama3_8b()
    cfg.max_seq = 1300
    model = rb.CausalLM(cfg).init_random(seed=26, std=0.02)
    defaults = {"qkv_post": "attention", "attention_merge": "launch"}
    try:
        for B, S in ((4, 1200), (32, 100)):
            prompt = np.random.default_rng(B).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)

            def run(**opts):
                for k, v in opts.items():
                    rb.set_option(k, v)
                try:
                    return _run(model, prompt, 5)
                finally:
                    for k, v in defaults.items():
                        rb.set_option(k, v)

            ids, logits = run()
            for opts in ({"qkv_post": "launch"}, {"attention_merge": "fused"}, {"qkv_post": "launch", "attention_merge": "fused"}):
                ids2, logits2 = run(**opts)
                assert np.array_equal(ids2, ids) and np.array_equal(logits2, logits), (B, S, opts)
    finally:
        model.free()


def test_full_size_continuous_batching_matches_the_plain_session(rb):
    """Llama-3-8B shape: four lanes over a pool of KV blocks, admitted in a scrambled order with another lane's
    admission and release in between (so the lanes' pages are interleaved in the pool), against a plain session with
    the same four prompts.  A lane's prefill is its prompt alone (300 rows: above the 256 rows up to which a Linear
    may split K, so its rows see the same sums as in the session's 1200-row prefill) and the decode steps see the
    same batch of four: same tokens, bit for bit; releasing the lanes returns every block."""
    cfg = W.llama3_8b()
    cfg.max_seq = 512
    model = rb.CausalLM(cfg).init_random(seed=27, std=0.02)
    try:
        B, S, steps = 4, 300, 6
        prompt = np.random.default_rng(10).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
        sess = model.session(B, S + steps + 8)
        want = sess.generate(prompt, steps)          # [B, steps]: first token from the prefill, then steps - 1 decode steps
        sess.free()
        ps = model.paged_session(B, S + steps + 8, 64)
        free0 = ps.free_blocks()
        first = {}
        first[2] = ps.admit(2, prompt[2])
        first[0] = ps.admit(0, prompt[0])
        ps.admit(3, prompt[1][:70])                  # a guest that leaves again: its pages return to the pool
        first[1] = ps.admit(1, prompt[1])
        ps.release(3)
        first[3] = ps.admit(3, prompt[3])
        got = ps.step(steps - 1)
        for b in range(B):
            assert first[b] == want[b, 0]
            assert np.array_equal(got[b], want[b, 1:])
        for b in range(B):
            ps.release(b)
        assert ps.free_blocks() == free0
        ps.free()
    finally:
        model.free()


@pytest.mark.parametrize("mode", ["top_k", "top_p"])
def test_full_size_sampling_follows_the_sequence_not_its_batch_slot(rb, mode):
    """Llama-3-8B shape (128 256-entry vocabulary), device sampling with a repetition penalty: a sequence's sampled
    tokens and log-probabilities depend on its own logits and its own key only, so permuting the batch together with
    the seeds permutes the results; eos and stop ids end a sequence (-1 afterwards) without disturbing the others."""
    cfg = W.llama3_8b()
    cfg.max_seq = 256
    model = rb.CausalLM(cfg).init_random(seed=28, std=0.02)
    try:
        B, S, steps = 8, 64, 6
        rng = np.random.default_rng(11)
        prompt = rng.integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
        seeds = np.arange(100, 100 + B, dtype=np.uint64)
        kw = dict(temperature=0.8, top_k=50, repetition_penalty=1.1) if mode == "top_k" else \
            dict(temperature=0.8, top_k=0, top_p=0.9, repetition_penalty=1.1)

        def run(p, sd, **gen):
            sess = model.session(B, S + steps + 8)
            sess.set_sampling(seeds=sd, **kw)
            ids = sess.generate(p, steps, **gen)
            lp = sess.logprobs(steps)
            sess.free()
            return ids, lp

        ids, lp = run(prompt, seeds)
        assert (ids >= 0).all() and (ids < cfg.vocab).all() and np.isfinite(lp).all() and (lp <= 0).all()
        perm = rng.permutation(B)
        ids_p, lp_p = run(prompt[perm], seeds[perm])
        assert np.array_equal(ids_p, ids[perm]) and np.array_equal(lp_p, lp[perm])
        other, _ = run(prompt, seeds + np.uint64(1000))
        assert not np.array_equal(other, ids)           # another key, another draw
        eos = int(ids[3, 2])
        stop = int(ids[5, 1])
        cut, _ = run(prompt, seeds, eos=eos, stop_ids=(stop,))
        for b in range(B):
            ends = [j for j in range(steps) if ids[b, j] in (eos, stop)]
            n = ends[0] + 1 if ends else steps
            assert np.array_equal(cut[b, :n], ids[b, :n]) and (cut[b, n:] == -1).all()
    finally:
        model.free()
