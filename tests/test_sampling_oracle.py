"""CPU checks of the oracle's random keys and samplers (src/rew/rng.nim, src/rew/infer/generate.nim:92-150).

The reference's own tests of rng.nim (tests/trng.nim) are property tests without golden values, so the
oracle is pinned here against a second, independent restatement in plain Python integers / numpy float32
written from the same source lines, plus those properties.
"""
import numpy as np
import pytest

from oracle import orc
from rew_b200 import weights

M32 = 0xFFFFFFFF


def py_threefry(ka, kb, ca, cb):
    """rng.nim:38-56: four rounds, rotations 13/15/26/6, parity 0x1BD11BDA."""
    k2 = ka ^ kb ^ 0x1BD11BDA
    x0, x1 = (ca + ka) & M32, (cb + kb) & M32
    for r in (13, 15, 26, 6):
        x0 = (x0 + x1) & M32
        x1 = ((x1 << r) | (x1 >> (32 - r))) & M32
        x1 ^= x0
    return (x0 + kb) & M32, (x1 + k2 + 1) & M32


def py_key(seed):
    return seed & M32, (seed >> 32) & M32


def py_fold(key, data):
    return py_threefry(key[0], key[1], data & M32, (data >> 32) & M32)


def py_uniform(key):
    return np.float32(py_fold(key, 0)[0] >> 8) * np.float32(1.0 / 16777216.0)


def py_sorted(logits):
    return sorted(range(len(logits)), key=lambda i: -float(logits[i]))  # stable: ties keep ascending index


def py_top_k(logits, k, key):
    order = py_sorted(logits)
    k = min(k, len(logits))
    probs = [np.exp(np.float32(logits[i])) for i in order[:k]]
    s = np.float32(0)
    for p in probs:
        s = np.float32(s + p)
    u, cum = py_uniform(key), np.float32(0)
    for j in range(k):
        cum = np.float32(cum + np.float32(probs[j] / s))
        if u <= cum:
            return order[j]
    return order[k - 1]


def py_top_p(logits, top_p, key):
    order = py_sorted(logits)
    mx = np.float32(logits[order[0]])
    probs = [np.exp(np.float32(np.float32(logits[i]) - mx)) for i in order]
    s = np.float32(0)
    for p in probs:
        s = np.float32(s + p)
    probs = [np.float32(p / s) for p in probs]
    cum, cutoff = np.float32(0), len(order)
    for j, p in enumerate(probs):
        cum = np.float32(cum + p)
        if cum >= np.float32(top_p):
            cutoff = j + 1
            break
    rn = np.float32(0)
    for p in probs[:cutoff]:
        rn = np.float32(rn + p)
    u, cum = py_uniform(key), np.float32(0)
    for j in range(cutoff):
        cum = np.float32(cum + np.float32(probs[j] / rn))
        if u <= cum:
            return order[j]
    return order[cutoff - 1]


def test_threefry_matches_independent_restatement():
    rng = np.random.default_rng(0)
    cases = [(0, 0, 0, 0), (M32, M32, M32, M32), (1, 0, 0, 0), (0, 0, 1, 0)]
    cases += [tuple(int(v) for v in rng.integers(0, 2**32, 4)) for _ in range(200)]
    for c in cases:
        assert orc.threefry(*c) == py_threefry(*c), c


def test_key_properties_as_the_reference_tests_them():
    # tests/trng.nim: different seeds differ, foldIn is deterministic and data-dependent
    a, b = orc.threefry(*py_key(11), 5, 0), orc.threefry(*py_key(11), 6, 0)
    assert a != b and a == orc.threefry(*py_key(11), 5, 0)
    hi = 0xCAFEBABE12345678
    assert py_key(hi) == (0x12345678, 0xCAFEBABE)
    us = [orc.uniform01(s) for s in range(64)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) > 60
    assert 0.3 < float(np.mean(us)) < 0.7


def test_uniform_with_folds():
    for seed in (0, 7, 2**40 + 3):
        k = py_key(seed)
        assert orc.uniform01(seed) == float(py_uniform(k))
        k2 = py_fold(py_fold(k, 0), 1)
        assert orc.uniform01(seed, [0, 1]) == float(py_uniform(k2))


@pytest.mark.parametrize("V,k", [(5, 3), (40, 50), (257, 16), (1000, 1)])
def test_sample_top_k(V, k):
    rng = np.random.default_rng(V)
    for seed in range(30):
        lg = rng.standard_normal(V).astype(np.float32) * 2
        lg[rng.integers(0, V, 3)] = lg[0]  # ties
        assert orc.sample_top_k(lg, k, seed) == py_top_k(lg, k, py_key(seed))


@pytest.mark.parametrize("V,p", [(5, 0.5), (64, 0.9), (300, 1.0), (300, 0.05)])
def test_sample_top_p(V, p):
    rng = np.random.default_rng(V + 1)
    for seed in range(30):
        lg = rng.standard_normal(V).astype(np.float32) * 3
        lg[rng.integers(0, V, 3)] = lg[1]
        assert orc.sample_top_p(lg, p, seed) == py_top_p(lg, p, py_key(seed))


def test_sampling_distribution_follows_softmax():
    lg = np.log(np.array([0.5, 0.25, 0.125, 0.125], np.float32))
    counts = np.zeros(4)
    for seed in range(4000):
        counts[orc.sample_top_p(lg, 1.0, seed)] += 1
    assert np.allclose(counts / 4000, [0.5, 0.25, 0.125, 0.125], atol=0.03)


def test_generate_sampled_greedy_settings_equal_generate_greedy():
    mc = weights.tiny_llama()
    ts = weights.init_weights(mc, seed=3)
    prompt = np.array([[1, 5, 9, 2], [3, 3, 7, 11]], np.int32)
    g, _ = orc.generate_greedy(mc, ts, prompt, 6)
    for kw in (dict(do_sample=False), dict(temperature=0.0), dict(top_k=1)):
        ids, lps = orc.generate_sampled(mc, ts, prompt, 6, **kw)
        assert np.array_equal(ids, g), kw
        assert np.all(lps <= 0) and np.all(np.isfinite(lps))


def test_generate_sampled_depends_on_seed_and_repeats():
    mc = weights.tiny_llama()
    ts = weights.init_weights(mc, seed=3)
    prompt = np.array([[1, 5, 9, 2]] * 4, np.int32)
    kw = dict(temperature=1.5, top_k=0, top_p=0.95)
    a, la = orc.generate_sampled(mc, ts, prompt, 8, seeds=[1, 1, 2, 3], **kw)
    b, lb = orc.generate_sampled(mc, ts, prompt, 8, seeds=[1, 1, 2, 3], **kw)
    assert np.array_equal(a, b) and np.array_equal(la, lb)
    assert np.array_equal(a[0], a[1])
    assert not (np.array_equal(a[0], a[2]) and np.array_equal(a[0], a[3]))
