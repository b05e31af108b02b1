"""CPU checks of the oracle's NF4 codec and QLoRA Linear against the reference's own test vector
(tests/teager_dispatch.nim:248-262, the same block in tests/tcore.nim:548 and tests/tjit_execute.nim:291)
and an independent numpy restatement of src/rew/quantize/codecs.nim:13-74."""
import numpy as np

from oracle import orc

TABLE = np.array([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                  -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                  0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                  0.7229568362236023, 1.0], np.float32)


def np_quantize(w, block):
    w = np.asarray(w, np.float32).reshape(-1)
    n = w.size
    nb = (n + block - 1) // block
    scales = np.empty(nb, np.float32)
    codes = np.empty(n, np.int64)
    for b in range(nb):
        seg = w[b * block:(b + 1) * block]
        am = np.float32(max(np.float32(1e-10), np.max(np.abs(seg))))
        scales[b] = am
        norm = np.clip(seg / am, np.float32(-1), np.float32(1)).astype(np.float32)
        codes[b * block:b * block + seg.size] = np.argmin(np.abs(norm[:, None] - TABLE[None, :]), axis=1)  # first min
    packed = np.zeros((n + 1) // 2, np.uint8)
    packed[:] = codes[0::2].astype(np.uint8)[: packed.size]
    odd = codes[1::2].astype(np.uint8)
    packed[: odd.size] |= odd << 4
    return packed, scales, codes


def test_reference_qlora_vector():
    # initQloraLinearFromF32(key, [1,0,0,1], 2, 2, bias=[0.5,-1], rank=1, alpha=1, groupSize=3); x = [[2,3]] -> [2.5, 2.0]
    packed, scales = orc.nf4_quantize([1.0, 0.0, 0.0, 1.0], 3)
    assert packed.size == 2 and scales.size == 2          # qweight.len == 2, qscales.len == 2
    rng = np.random.default_rng(0)
    A = rng.uniform(-0.7, 0.7, size=(1, 2)).astype(np.float32)     # B starts at zero, so A does not matter
    y = orc.qlora_forward([[2.0, 3.0]], packed, scales, 2, 2, 3, bias=[0.5, -1.0], A=A, B=np.zeros((2, 1)), scaling=1.0)
    assert np.allclose(y, [[2.5, 2.0]], atol=1e-6)


def test_quantize_matches_numpy_restatement_bit_for_bit():
    rng = np.random.default_rng(1)
    for n, block in ((64, 64), (1000, 64), (129, 32), (4, 3), (7, 64)):
        w = (rng.standard_normal(n) * rng.uniform(0.01, 3)).astype(np.float32)
        w[rng.integers(0, n)] = 0.0
        p, s = orc.nf4_quantize(w, block)
        p2, s2, codes = np_quantize(w, block)
        assert np.array_equal(p, p2) and np.array_equal(s, s2)
        deq = orc.nf4_dequantize(p, s, n, block)
        assert np.array_equal(deq, TABLE[codes] * np.repeat(s2, block)[:n])
        # per-block absmax scaling: the error is bounded by half the widest table gap times the scale
        assert np.all(np.abs(deq - w) <= 0.16 * np.repeat(s2, block)[:n] + 1e-7)


def test_all_zero_block_and_extremes():
    p, s = orc.nf4_quantize(np.zeros(64, np.float32), 64)
    assert np.all(s == np.float32(1e-10)) and np.all(p == 0x77)        # code 7 = 0.0 in both nibbles
    w = np.array([2.0, -2.0, 1.0, -1.0], np.float32)
    p, s = orc.nf4_quantize(w, 4)
    # 1.0 -> 15, -1.0 -> 0; 0.5 is nearer to 0.4407 (12) than to 0.5626 (13); -0.5 -> -0.5251 (2)
    assert s[0] == 2.0 and p.tolist() == [0x0F, 0x2C]
