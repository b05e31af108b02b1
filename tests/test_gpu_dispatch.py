"""Tier-A per-op dispatch (the EagerBackend slot as a C call) against the reference's own
known-answer vectors (tests/teager_dispatch.nim) and numpy."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rb():
    from rew_b200 import _lib, api
    _lib.init()
    return api


def T(rb, a, dtype=None):
    return rb.Tensor.from_host(a, dtype)


def D(rb, op, operands, **attrs):
    return [t.to_host() for t in rb.dispatch(op, operands, [(k, v) for k, v in attrs.items()])]


A = np.array([1, 2, 3, 4], np.float32)
B = np.array([10, 20, 30, 40], np.float32)


def test_reference_pinned_vectors(rb):
    a, b = T(rb, A), T(rb, B)
    assert D(rb, "add", [a, b])[0].tolist() == [11.0, 22.0, 33.0, 44.0]           # teager_dispatch.nim:264-267
    assert D(rb, "mul", [a, b])[0].tolist() == [10.0, 40.0, 90.0, 160.0]          # :269-272
    assert D(rb, "neg", [a])[0].tolist() == [-1.0, -2.0, -3.0, -4.0]              # :281-284
    np.testing.assert_allclose(D(rb, "exp", [a])[0], np.exp(A), rtol=1e-6)         # :286-291
    np.testing.assert_allclose(D(rb, "logistic", [a])[0], 1 / (1 + np.exp(-A)), atol=1e-4)  # :338-343
    assert D(rb, "reshape", [a], shape="[2,2]")[0].tolist() == [[1.0, 2.0], [3.0, 4.0]]     # :543-547
    m1 = rb.dispatch("reshape", [a], [("shape", "@[2, 2]")])[0]                   # both int-list spellings parse
    m2 = rb.dispatch("reshape", [b], [("shape", "[2,2]")])[0]
    assert D(rb, "transpose", [m1], permutation="@[1, 0]")[0].ravel().tolist() == [1.0, 3.0, 2.0, 4.0]  # :549-554
    assert D(rb, "reduceSum", [a], dims="[0]")[0].tolist() == 10.0                # :562-566
    got = D(rb, "dotGeneral", [m1, m2], lhs_batching="[]", rhs_batching="[]", lhs_contracting="[1]", rhs_contracting="[0]")[0]
    assert got.ravel().tolist() == [70.0, 100.0, 150.0, 220.0]                     # :584-598
    s = T(rb, np.array([5.0], np.float32))
    assert D(rb, "broadcastTo", [s], output_shape="[3]", broadcast_dimensions="[0]")[0].tolist() == [5.0, 5.0, 5.0]  # :600-605
    assert D(rb, "iota", [], dtype="int32", shape="[2,3]", dimension="1")[0].ravel().tolist() == [0, 1, 2, 0, 1, 2]  # :505-509
    i = T(rb, np.array([1, 2, 3], np.int32))
    assert D(rb, "astype", [i], dtype="float32")[0].tolist() == [1.0, 2.0, 3.0]   # :408-411


def test_layout_ops_against_numpy(rb):
    rng = np.random.default_rng(0)
    x = rng.normal(size=(2, 3, 4, 5)).astype(np.float32)
    t = T(rb, x)
    assert np.array_equal(D(rb, "transpose", [t], permutation="[0,2,1,3]")[0], x.transpose(0, 2, 1, 3))
    assert np.array_equal(D(rb, "slice", [t], start_indices="[0,1,0,1]", limit_indices="[2,3,4,5]", strides="[1,1,2,2]")[0],
                          x[:, 1:3, ::2, 1::2])
    y = rng.normal(size=(2, 3, 2, 5)).astype(np.float32)
    assert np.array_equal(D(rb, "concat", [t, T(rb, y)], dimension="2")[0], np.concatenate([x, y], 2))
    v = rng.normal(size=(3, 5)).astype(np.float32)
    got = D(rb, "broadcastTo", [T(rb, v)], output_shape="[2,3,4,5]", broadcast_dimensions="[1,3]")[0]
    assert np.array_equal(got, np.broadcast_to(v[None, :, None, :], (2, 3, 4, 5)))
    np.testing.assert_allclose(D(rb, "reduceSum", [t], dims="[1,3]")[0], x.sum((1, 3)), rtol=1e-5)
    assert np.array_equal(D(rb, "reduceMax", [t], dims="[3]")[0], x.max(3))


def test_compare_select_and_causal_mask_composition(rb):
    """makeCausalMask exactly as rew composes it (src/rew/nn/attention.nim:18-34)."""
    rows = rb.dispatch("iota", [], [("dtype", "int32"), ("shape", "[4, 4]"), ("dimension", "0")])[0]
    cols = rb.dispatch("iota", [], [("dtype", "int32"), ("shape", "[4, 4]"), ("dimension", "1")])[0]
    upper = rb.dispatch("compare", [rows, cols], [("comparison_direction", "LE")])[0]
    neg = T(rb, np.full((4, 4), -1e9, np.float32))
    zero = T(rb, np.zeros((4, 4), np.float32))
    mask = rb.dispatch("select", [upper, zero, neg])[0].to_host()
    want = np.where(np.arange(4)[:, None] <= np.arange(4)[None, :], 0.0, -1e9).astype(np.float32)
    assert np.array_equal(mask, want)


def test_batched_dot_general_and_topk(rb):
    rng = np.random.default_rng(1)
    q = rng.normal(size=(2, 3, 5, 8)).astype(np.float32)
    k = rng.normal(size=(2, 3, 7, 8)).astype(np.float32)
    got = D(rb, "dotGeneral", [T(rb, q), T(rb, k)], lhs_batching="[0,1]", rhs_batching="[0,1]", lhs_contracting="[3]",
            rhs_contracting="[3]")[0]
    np.testing.assert_allclose(got, q @ k.transpose(0, 1, 3, 2), rtol=1e-5, atol=1e-5)
    p = rng.normal(size=(6, 64)).astype(np.float32)
    p[0, 10] = p[0, 20]  # an exact tie keeps ascending index order
    vals, idx = D(rb, "topK", [T(rb, p)], k="6")
    order = np.argsort(-p, axis=-1, kind="stable")[:, :6]
    assert np.array_equal(idx, order.astype(np.int32))
    assert np.array_equal(vals, np.take_along_axis(p, order, -1))


def test_dispatch_errors(rb):
    from rew_b200._lib import RewB200Error
    a = T(rb, A)
    with pytest.raises(RewB200Error, match="not supported"):
        rb.dispatch("conv2d", [a])
    with pytest.raises(RewB200Error, match="shape mismatch"):
        rb.dispatch("add", [a, T(rb, np.zeros(3, np.float32))])
    with pytest.raises(RewB200Error, match="only float32"):
        rb.dispatch("reduceSum", [T(rb, np.zeros(3, np.int32))], [("dims", "[0]")])
    with pytest.raises(RewB200Error, match="missing attribute"):
        rb.dispatch("transpose", [a])
