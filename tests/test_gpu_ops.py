"""GPU parity of the Tier-B entry points against the CPU oracle, through the C ABI.

f32: rel-L2 <= 1e-5 (the north star's fp32 bar).  bf16: the oracle runs in f32
on bf16-rounded inputs and the result is compared at rel-L2 <= 2e-2.
"""
import os

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")
F32_TOL = 1e-5
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def rb():
    from rew_b200 import _lib, api
    _lib.init()
    return api


def T(rb, a, dtype=None):
    return rb.Tensor.from_host(a, dtype)


def test_buffer_roundtrip_and_release(rb):
    from rew_b200 import _lib
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    t = T(rb, x)
    assert t.shape == (2, 3, 4) and t.dtype == _lib.F32
    assert np.array_equal(t.to_host(), x)
    t.release()
    t.release()  # idempotent, nil-safe (buffer.nim:69-82)
    ids = np.array([[1, 2], [3, 4]], np.int32)
    assert np.array_equal(T(rb, ids).to_host(), ids)
    e = T(rb, np.zeros((0, 4), np.float32))  # empty
    assert e.to_host().shape == (0, 4)
    b = T(rb, x, _lib.BF16)
    assert np.array_equal(b.to_host(), x)  # small integers are exact in bf16


def test_golden_small_ops_f32(rb, orc):
    z = np.load(os.path.join(GOLD, "small_ops.npz"))
    x = T(rb, z["lin_x"])
    lin = rb.Linear(T(rb, z["lin_w"]), T(rb, z["lin_b"]))
    assert rel_l2(lin.forward(x).to_host(), z["lin_y"]) < F32_TOL
    assert rel_l2(rb.rmsNorm(x, T(rb, z["norm_g"]), 1e-5).to_host(), z["rms_y"]) < F32_TOL
    ln = rb.LayerNorm(T(rb, z["norm_g"]), T(rb, z["norm_b"]), 1e-5)
    assert rel_l2(ln.forward(x).to_host(), z["ln_y"]) < F32_TOL
    rope = rb.RotaryPositionEncoding(16, 32, 10000.0)
    assert np.array_equal(rope.cosCached.to_host(), z["rope_cos"])  # host tables, bit-equal
    assert np.array_equal(rope.sinCached.to_host(), z["rope_sin"])
    assert rel_l2(rope.forward(T(rb, z["rope_x"]), 5).to_host(), z["rope_y"]) < F32_TOL
    q, k, v = T(rb, z["att_q"]), T(rb, z["att_k"]), T(rb, z["att_v"])
    assert rel_l2(rb.scaledDotProductAttention(q, k, v, False).to_host(), z["att_plain"]) < F32_TOL
    assert rel_l2(rb.scaledDotProductAttention(q, k, v, True, 0).to_host(), z["att_as_written"]) < F32_TOL
    assert rel_l2(rb.scaledDotProductAttention(q, k, v, True, 1).to_host(), z["att_standard"]) < F32_TOL
    ffn = rb.GatedFeedForward(rb.Linear(T(rb, z["ffn_gw"]), T(rb, z["ffn_gb"])),
                              rb.Linear(T(rb, z["ffn_uw"]), T(rb, z["ffn_ub"])),
                              rb.Linear(T(rb, z["ffn_dw"]), T(rb, z["ffn_db"])))
    assert rel_l2(ffn.forward(x).to_host(), z["ffn_y"]) < F32_TOL


def test_pinned_reference_matmul_vector(rb):
    # tests/teager_dispatch.nim:584-598
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[10, 20], [30, 40]], np.float32)
    y = rb.Linear(T(rb, b), T(rb, np.zeros(2, np.float32))).forward(T(rb, a)).to_host()
    assert y.ravel().tolist() == [70.0, 100.0, 150.0, 220.0]


@pytest.mark.parametrize("M,K,N", [(1, 64, 8), (3, 72, 40), (32, 4096, 1024), (7, 688, 256), (32, 256, 1376),
                                   (33, 128, 136), (200, 320, 264)])
def test_linear_bf16_shapes(rb, orc, M, K, N):
    from rew_b200 import _lib
    rng = np.random.default_rng(M * 1000 + N)
    x = orc.bf16_round(rng.normal(size=(M, K)))
    w = orc.bf16_round(rng.normal(0, 0.05, size=(K, N)))
    b = rng.normal(0, 0.1, size=(N,)).astype(np.float32)
    want = orc.linear(x, w, b)
    got = rb.Linear(T(rb, w, _lib.BF16), T(rb, b)).forward(T(rb, x, _lib.BF16)).to_host()
    assert got.shape == (M, N)
    assert rel_l2(got, want) < 5e-3  # only the bf16 rounding of the output


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (5, 17, 3), (64, 64, 64), (70, 130, 65)])
def test_linear_f32_shapes(rb, orc, M, K, N):
    rng = np.random.default_rng(K)
    x = rng.normal(size=(M, K)).astype(np.float32)
    w = rng.normal(size=(K, N)).astype(np.float32)
    b = rng.normal(size=(N,)).astype(np.float32)
    got = rb.Linear(T(rb, w), T(rb, b)).forward(T(rb, x)).to_host()
    assert rel_l2(got, orc.linear(x, w, b)) < F32_TOL


def test_linear_errors_follow_reference_wording(rb):
    from rew_b200._lib import RewB200Error
    x = T(rb, np.zeros((2, 3), np.float32))
    w = T(rb, np.zeros((4, 5), np.float32))
    with pytest.raises(RewB200Error, match="matmul: inner dim mismatch"):
        rb.Linear(w, None).forward(x)
    with pytest.raises(RewB200Error, match="rank-2"):
        rb.Linear(w, None).forward(T(rb, np.zeros((2, 2, 4), np.float32)))


@pytest.mark.parametrize("rows,d", [(1, 8), (5, 256), (32, 4096), (3, 8192)])
def test_norms(rb, orc, rows, d):
    from rew_b200 import _lib
    rng = np.random.default_rng(d)
    x = rng.normal(size=(rows, d)).astype(np.float32) * 3
    g = (1 + 0.1 * rng.normal(size=d)).astype(np.float32)
    b = (0.1 * rng.normal(size=d)).astype(np.float32)
    assert rel_l2(rb.rmsNorm(T(rb, x), T(rb, g), 1e-5).to_host(), orc.rmsnorm(x, g, 1e-5)) < F32_TOL
    assert rel_l2(rb.LayerNorm(T(rb, g), T(rb, b), 1e-5).forward(T(rb, x)).to_host(), orc.layernorm(x, g, b, 1e-5)) < F32_TOL
    xb = orc.bf16_round(x)
    assert rel_l2(rb.rmsNorm(T(rb, xb, _lib.BF16), T(rb, g), 1e-5).to_host(), orc.rmsnorm(xb, g, 1e-5)) < 5e-3


def test_rope_bf16_and_errors(rb, orc):
    from rew_b200 import _lib
    from rew_b200._lib import RewB200Error
    rope = rb.RotaryPositionEncoding(128, 64, 500000.0)
    c, s = orc.rope_tables(128, 64, 500000.0)
    x = orc.bf16_round(np.random.default_rng(0).normal(size=(2, 4, 7, 128)))
    got = rope.forward(T(rb, x, _lib.BF16), 11).to_host()
    assert rel_l2(got, orc.rope_apply(x, c, s, 11)) < 5e-3
    with pytest.raises(RewB200Error, match="exceeds maxSeqLen"):
        rope.forward(T(rb, x, _lib.BF16), 60)
    with pytest.raises(RewB200Error, match="headDim mismatch"):
        rope.forward(T(rb, np.zeros((1, 2, 64), np.float32)), 0)


@pytest.mark.parametrize("B,nh,kvh,S,L,hd", [(1, 2, 1, 1, 1, 8), (2, 8, 2, 5, 5, 32), (1, 4, 4, 1, 70, 32),
                                             (2, 4, 2, 3, 130, 64), (1, 2, 2, 4, 4, 256)])
@pytest.mark.parametrize("mode", ["plain", "as_written", "standard"])
def test_attention_f32(rb, orc, B, nh, kvh, S, L, hd, mode):
    rng = np.random.default_rng(L * 7 + S)
    q = rng.normal(size=(B, nh, S, hd)).astype(np.float32)
    k = rng.normal(size=(B, kvh, L, hd)).astype(np.float32)
    v = rng.normal(size=(B, kvh, L, hd)).astype(np.float32)
    causal, mk = {"plain": (False, 0), "as_written": (True, 0), "standard": (True, 1)}[mode]
    got = rb.scaledDotProductAttention(T(rb, q), T(rb, k), T(rb, v), causal, mk).to_host()
    assert rel_l2(got, orc.gqa_attention(q, k, v, causal, mk)) < F32_TOL


@pytest.mark.parametrize("B,nh,kvh,L,hd", [(2, 8, 2, 1, 128), (3, 8, 2, 63, 128), (2, 32, 8, 64, 128),
                                           (4, 8, 1, 257, 128), (1, 16, 16, 100, 128), (2, 4, 2, 200, 64),
                                           (40, 8, 8, 130, 128)])
def test_attention_bf16_decode(rb, orc, B, nh, kvh, L, hd):
    from rew_b200 import _lib
    rng = np.random.default_rng(L)
    q = orc.bf16_round(rng.normal(size=(B, nh, 1, hd)))
    k = orc.bf16_round(rng.normal(size=(B, kvh, L, hd)))
    v = orc.bf16_round(rng.normal(size=(B, kvh, L, hd)))
    got = rb.scaledDotProductAttention(T(rb, q, _lib.BF16), T(rb, k, _lib.BF16), T(rb, v, _lib.BF16), True, 1).to_host()
    assert rel_l2(got, orc.gqa_attention(q, k, v, True, 1)) < BF16_TOL


def test_attention_bf16_decode_fused_merge_equals_merge_launch(rb, orc):
    """Split-KV decode: a second launch combines the splits; with option attention_merge=fused the last CTA
    of a (sequence, kv head) does it inside the kernel.  Same partials, same arithmetic: equal bits.
    Run twice so that the arrival counters are shown to return to zero."""
    from rew_b200 import _lib
    rng = np.random.default_rng(77)
    B, nh, kvh, L, hd = 3, 8, 2, 1000, 128
    q = orc.bf16_round(rng.normal(size=(B, nh, 1, hd)))
    k = orc.bf16_round(rng.normal(size=(B, kvh, L, hd)))
    v = orc.bf16_round(rng.normal(size=(B, kvh, L, hd)))
    tq, tk, tv = T(rb, q, _lib.BF16), T(rb, k, _lib.BF16), T(rb, v, _lib.BF16)
    two = rb.scaledDotProductAttention(tq, tk, tv, True, 1).to_host()
    rb.set_option("attention_merge", "fused")
    try:
        fused = [rb.scaledDotProductAttention(tq, tk, tv, True, 1).to_host() for _ in range(2)]
    finally:
        rb.set_option("attention_merge", "launch")
    assert np.array_equal(fused[0], two) and np.array_equal(fused[1], two)
    assert rel_l2(two, orc.gqa_attention(q, k, v, True, 1)) < BF16_TOL


@pytest.mark.parametrize("B,nh,kvh,S,hd", [(1, 4, 2, 2, 128), (2, 8, 2, 64, 128), (1, 4, 1, 150, 128), (2, 4, 4, 65, 64)])
@pytest.mark.parametrize("mode", ["plain", "as_written", "standard"])
def test_attention_bf16_prefill(rb, orc, B, nh, kvh, S, hd, mode):
    from rew_b200 import _lib
    rng = np.random.default_rng(S)
    q = orc.bf16_round(rng.normal(size=(B, nh, S, hd)))
    k = orc.bf16_round(rng.normal(size=(B, kvh, S, hd)))
    v = orc.bf16_round(rng.normal(size=(B, kvh, S, hd)))
    causal, mk = {"plain": (False, 0), "as_written": (True, 0), "standard": (True, 1)}[mode]
    got = rb.scaledDotProductAttention(T(rb, q, _lib.BF16), T(rb, k, _lib.BF16), T(rb, v, _lib.BF16), causal, mk).to_host()
    assert rel_l2(got, orc.gqa_attention(q, k, v, causal, mk)) < BF16_TOL


def test_attention_config2_bf16_decode_shape(rb, orc):
    """The attention-operator configuration, decode: batch 8, 32 q / 8 kv heads, head_dim 128, one query over a
    cache of 4096 per sequence; every sequence against the oracle."""
    from rew_b200 import _lib
    rng = np.random.default_rng(42)
    B, nh, kvh, L, hd = 8, 32, 8, 4096, 128
    q = orc.bf16_round(rng.normal(size=(B, nh, 1, hd)))
    k = orc.bf16_round(rng.normal(size=(B, kvh, L, hd)))
    v = orc.bf16_round(rng.normal(size=(B, kvh, L, hd)))
    got = rb.scaledDotProductAttention(T(rb, q, _lib.BF16), T(rb, k, _lib.BF16), T(rb, v, _lib.BF16), True, 1).to_host()
    want = orc.gqa_attention(q, k, v, True, 1)
    assert rel_l2(got, want) < BF16_TOL
    assert max(rel_l2(got[b], want[b]) for b in range(B)) < BF16_TOL


def test_attention_config2_bf16_prefill_shape(rb, orc):
    """The attention-operator configuration, prefill: batch 8, 32 q / 8 kv heads, head_dim 128, causal, 4096
    positions (32 key tiles per query block on the tcgen05 kernel).  The device computes all of it; the oracle
    (O(S^2) per head) checks the first and the last kv group of one sequence in the middle of the batch and
    the first kv group of the last sequence: 12 of 256 query heads, all 4096 rows of each."""
    from rew_b200 import _lib
    rng = np.random.default_rng(43)
    B, nh, kvh, S, hd = 8, 32, 8, 4096, 128
    q = orc.bf16_round(rng.standard_normal(size=(B, nh, S, hd), dtype=np.float32))
    k = orc.bf16_round(rng.standard_normal(size=(B, kvh, S, hd), dtype=np.float32))
    v = orc.bf16_round(rng.standard_normal(size=(B, kvh, S, hd), dtype=np.float32))
    args = (T(rb, q, _lib.BF16), T(rb, k, _lib.BF16), T(rb, v, _lib.BF16), True, 1)
    got = rb.scaledDotProductAttention(*args).to_host()     # 4096 rows: two query tiles per CTA
    assert np.isfinite(got).all()
    rb.set_option("attention", "tc1")
    try:
        one_tile = rb.scaledDotProductAttention(*args).to_host()
    finally:
        rb.set_option("attention", "tc")
    assert np.array_equal(got, one_tile)
    g = nh // kvh
    for b, groups in ((3, (0, kvh - 1)), (B - 1, (0,))):
        heads = np.concatenate([np.arange(kg * g, (kg + 1) * g) for kg in groups])
        want = orc.gqa_attention(np.ascontiguousarray(q[b:b + 1, heads]), np.ascontiguousarray(k[b:b + 1, list(groups)]),
                                 np.ascontiguousarray(v[b:b + 1, list(groups)]), True, 1)
        assert rel_l2(got[b:b + 1, heads], want) < BF16_TOL
        # early rows see few keys and late rows all of them: check both ends on their own
        assert rel_l2(got[b:b + 1, heads, :128], want[:, :, :128]) < BF16_TOL
        assert rel_l2(got[b:b + 1, heads, -128:], want[:, :, -128:]) < BF16_TOL


def test_swiglu_and_embedding(rb, orc):
    from rew_b200 import _lib
    from rew_b200._lib import RewB200Error
    rng = np.random.default_rng(9)
    x = orc.bf16_round(rng.normal(size=(6, 64)))
    gw, uw = (orc.bf16_round(rng.normal(0, 0.1, size=(64, 48))) for _ in range(2))
    dw = orc.bf16_round(rng.normal(0, 0.1, size=(48, 64)))
    zb = lambda n: np.zeros(n, np.float32)
    ffn = rb.GatedFeedForward(rb.Linear(T(rb, gw, _lib.BF16), T(rb, zb(48))), rb.Linear(T(rb, uw, _lib.BF16), T(rb, zb(48))),
                              rb.Linear(T(rb, dw, _lib.BF16), T(rb, zb(64))))
    got = ffn.forward(T(rb, x, _lib.BF16)).to_host()
    assert rel_l2(got, orc.gated_ffn(x, gw, zb(48), uw, zb(48), dw, zb(64))) < BF16_TOL
    table = rng.normal(size=(50, 16)).astype(np.float32)
    ids = rng.integers(0, 50, size=(3, 4)).astype(np.int32)
    emb = rb.Embedding(T(rb, table))
    got = emb.forward(T(rb, ids)).to_host()
    assert got.shape == (3, 4, 16)
    assert np.array_equal(got, orc.embedding_onehot(ids, table))  # gather == one-hot matmul, exactly
    bad = T(rb, np.array([51], np.int32))
    with pytest.raises(RewB200Error, match="out of range"):
        emb.forward(bad).to_host()


@pytest.mark.parametrize("B,nh,kvh,S,L", [(2, 8, 2, 512, 512), (1, 4, 4, 300, 300), (1, 8, 1, 130, 400), (3, 4, 2, 128, 128),
                                          (1, 2, 2, 1000, 1000), (2, 4, 2, 256, 256), (1, 4, 1, 384, 700)])
@pytest.mark.parametrize("mode", ["plain", "standard"])
def test_attention_bf16_prefill_tcgen05(rb, orc, B, nh, kvh, S, L, mode):
    """head_dim 128 and at least 128 queries: the tcgen05 kernel (S and O in tensor memory).  Ragged last
    tiles, grouped heads, and a context longer than the query block (keys j <= i + L - S visible)."""
    from rew_b200 import _lib
    rng = np.random.default_rng(S + L)
    q = orc.bf16_round(rng.normal(size=(B, nh, S, 128)))
    k = orc.bf16_round(rng.normal(size=(B, kvh, L, 128)))
    v = orc.bf16_round(rng.normal(size=(B, kvh, L, 128)))
    causal, mk = {"plain": (False, 0), "standard": (True, 1)}[mode]
    args = (T(rb, q, _lib.BF16), T(rb, k, _lib.BF16), T(rb, v, _lib.BF16), causal, mk)
    got = rb.scaledDotProductAttention(*args).to_host()
    want = orc.gqa_attention(q, k, v, causal, mk)
    assert rel_l2(got, want) < BF16_TOL
    rb.set_option("attention", "mma")
    try:
        ref = rb.scaledDotProductAttention(*args).to_host()
        rb.set_option("attention", "tc2")
        two_tiles = rb.scaledDotProductAttention(*args).to_host()
    finally:
        rb.set_option("attention", "tc")
    assert rel_l2(got, ref) < 1e-2   # two correct bf16 kernels agree far inside the tolerance
    # one query tile per CTA (the default at these sizes) and two query tiles per CTA (forced from 256 query rows
    # up) do the same arithmetic per row
    assert np.array_equal(got, two_tiles)
