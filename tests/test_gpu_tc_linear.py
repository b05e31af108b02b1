"""The tcgen05 / tensor-memory Linear against the oracle and against the mma.sync Linear,
through the C ABI (option "linear" = "tc")."""
import numpy as np
import pytest

from conftest import rel_l2
from rew_b200 import weights as W

pytestmark = pytest.mark.gpu


@pytest.fixture()
def rb_tc():
    from rew_b200 import _lib, api
    _lib.init()
    api.set_option("linear", "tc")
    yield api
    api.set_option("linear", "tc")  # the default


@pytest.mark.parametrize("M,K,N", [(1, 64, 8), (32, 64, 128), (32, 4096, 1024), (7, 688, 256), (32, 256, 1376),
                                   (33, 128, 136), (64, 512, 256), (100, 320, 264), (128, 1024, 384),
                                   (200, 320, 264), (256, 2048, 512), (300, 576, 640)])
def test_tc_linear_shapes(rb_tc, orc, M, K, N):
    from rew_b200 import _lib
    rng = np.random.default_rng(M * 1000 + N)
    x = orc.bf16_round(rng.normal(size=(M, K)))
    w = orc.bf16_round(rng.normal(0, 0.05, size=(K, N)))
    b = rng.normal(0, 0.1, size=(N,)).astype(np.float32)
    want = orc.linear(x, w, b)
    T = rb_tc.Tensor.from_host
    got = rb_tc.Linear(T(w, _lib.BF16), T(b)).forward(T(x, _lib.BF16)).to_host()
    assert got.shape == (M, N)
    assert rel_l2(got, want) < 5e-3


def test_tc_model_matches_oracle_and_mma_path(rb_tc, orc):
    """Whole bf16 model on the tcgen05 Linear: split-K partial, SwiGLU and f32-logit epilogues."""
    from rew_b200 import _lib
    cfg = W.ModelConfig(vocab=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64, ffn=688, max_seq=256,
                        theta=500000.0, dtype=_lib.BF16, mask_kind=1)
    t = [orc.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(cfg, seed=4, std=0.05, trivial_affine=False)]
    for B, S in ((3, 70), (32, 16), (2, 150)):
        prompt = np.random.default_rng(B).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
        sess = rb_tc.CausalLM(cfg).load(t).session(B, S + 8)
        nxt, logits = sess.forward(prompt, want_logits=True)
        want = orc.model_forward(cfg, t, prompt, 0, True)[:, -1]
        assert rel_l2(logits, want) <= 2e-2
        ids, last = sess.decode(3, want_logits=True)
        seq = np.concatenate([prompt, nxt[:, None], ids[:, :2]], 1)
        want = orc.model_forward(cfg, t, seq, 0, True)[:, -1]
        assert rel_l2(last, want) <= 2e-2
        rb_tc.set_option("linear", "mma")
        sess2 = rb_tc.CausalLM(cfg).load(t).session(B, S + 8)
        _, logits_mma = sess2.forward(prompt, want_logits=True)
        rb_tc.set_option("linear", "tc")
        assert rel_l2(logits, logits_mma) <= 1e-2


def test_persistent_prefill_linear_matches_oracle(rb_tc, orc):
    """Enough 256-token tiles (17 x 20 >= 2 per SM) for the persistent kernel with the double-buffered
    accumulator; a ragged last token tile and a last feature tile that is only half there."""
    from rew_b200 import _lib
    M, K, N = 4100, 320, 2496
    rng = np.random.default_rng(11)
    x = orc.bf16_round(rng.normal(size=(M, K)))
    w = orc.bf16_round(rng.normal(0, 0.05, size=(K, N)))
    b = rng.normal(0, 0.1, size=(N,)).astype(np.float32)
    want = orc.linear(x, w, b)
    T = rb_tc.Tensor.from_host
    lin = rb_tc.Linear(T(w, _lib.BF16), T(b))
    got = lin.forward(T(x, _lib.BF16)).to_host()
    assert rel_l2(got, want) < 5e-3
    rb_tc.set_option("prefill", "tile")
    try:
        again = lin.forward(T(x, _lib.BF16)).to_host()
    finally:
        rb_tc.set_option("prefill", "pair")
    assert np.array_equal(got, again)   # same MMA order, same rounding: the two kernels agree bit for bit


@pytest.mark.parametrize("M,K,N,epi_bias", [(4100, 320, 2560, True), (8192, 1024, 1024, False), (5000, 64, 512, True)])
def test_pair_prefill_linear_matches_oracle_and_the_one_cta_kernels(rb_tc, orc, M, K, N, epi_bias):
    """Widths that are multiples of 256 with at least two 256-token tiles per SM run on pairs of CTAs
    (tcgen05 cta_group::2, 256 x 256 tiles, each CTA staging half of either operand).  Ragged last token tile,
    a single 64-row k block, more tiles than pairs: against the oracle, and bit for bit against the one-CTA
    persistent kernel and the one-tile kernel (the same k order and the same rounding)."""
    from rew_b200 import _lib
    rng = np.random.default_rng(M + N)
    x = orc.bf16_round(rng.normal(size=(M, K)))
    w = orc.bf16_round(rng.normal(0, 0.05, size=(K, N)))
    b = rng.normal(0, 0.1, size=(N,)).astype(np.float32) if epi_bias else np.zeros(N, np.float32)
    want = orc.linear(x, w, b)
    T = rb_tc.Tensor.from_host
    lin = rb_tc.Linear(T(w, _lib.BF16), T(b))
    got = lin.forward(T(x, _lib.BF16)).to_host()
    assert rel_l2(got, want) < 5e-3
    assert max(rel_l2(got[r], want[r]) for r in (0, 127, 128, 255, 256, M // 2, M - 1)) < 2e-2
    others = {}
    for how in ("persistent", "tile"):
        rb_tc.set_option("prefill", how)
        try:
            others[how] = lin.forward(T(x, _lib.BF16)).to_host()
        finally:
            rb_tc.set_option("prefill", "pair")
    assert np.array_equal(others["persistent"], others["tile"])
    assert np.array_equal(got, others["persistent"])


def test_persistent_prefill_model_equals_tile_kernel(rb_tc):
    """A 20 480-token prefill puts every decoder Linear (f32 partial, SwiGLU and bf16 epilogues) on the
    persistent kernel; the logits must equal those of the one-tile-per-CTA kernel exactly."""
    from rew_b200 import _lib
    cfg = W.ModelConfig(vocab=512, d_model=512, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1408, max_seq=640,
                        theta=500000.0, dtype=_lib.BF16, mask_kind=1)
    model = rb_tc.CausalLM(cfg).init_random(seed=3, std=0.05)
    B, S = 40, 512
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
    sess = model.session(B, S + 8)
    _, a = sess.forward(prompt, want_logits=True)
    rb_tc.set_option("prefill", "tile")
    try:
        sess.reset()
        _, b = sess.forward(prompt, want_logits=True)
    finally:
        rb_tc.set_option("prefill", "pair")
    assert np.isfinite(a).all() and np.array_equal(a, b)
