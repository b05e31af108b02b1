"""GPU parity of the NF4 weight-only Linear with the oracle's restatement of nf4Quantize / nf4Dequantize
(src/rew/quantize/codecs.nim:13-70) and QloraLinear.forward (src/rew/nn/lora.nim:410-431): the codes and
scales bit for bit, the projection within the bf16 tolerance (rel-L2 <= 2e-2)."""
import numpy as np
import pytest

from conftest import rel_l2
from rew_b200 import _lib
from rew_b200.weights import from_bf16_bits, to_bf16_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rb():
    from rew_b200 import api
    _lib.init()
    return api


def bf16_round(a):
    return from_bf16_bits(to_bf16_bits(np.asarray(a, np.float32)))


@pytest.mark.parametrize("K,N,src", [(64, 64, "f32"), (256, 192, "f32"), (512, 1024, "bf16"), (1024, 128, "bf16")])
def test_codes_and_scales_bit_exact(rb, orc, K, N, src):
    rng = np.random.default_rng(K + N)
    w = (rng.standard_normal((K, N)) * rng.uniform(0.01, 0.2, size=(K, 1))).astype(np.float32)
    w[rng.integers(0, K, 8), rng.integers(0, N, 8)] = 0.0
    if src == "bf16":
        w = bf16_round(w)
    layer = rb.QloraLinear(rb.Tensor.from_host(w, dtype=_lib.BF16 if src == "bf16" else _lib.F32))
    packed, scales = layer.unpack()
    want_p, want_s = orc.nf4_quantize(w, 64)
    assert np.array_equal(scales, want_s)
    assert np.array_equal(packed, want_p)
    # dequantised weight = level * scale rounded to bf16
    deq = layer.dequantized_weight().to_host()
    assert np.array_equal(deq, bf16_round(orc.nf4_dequantize(want_p, want_s, K * N, 64).reshape(K, N)))


@pytest.mark.parametrize("M,K,N", [(1, 256, 128), (1, 4096, 1024), (2, 512, 192), (3, 1024, 1024), (4, 4096, 512), (7, 512, 1024),
                                   (16, 1024, 256), (32, 4096, 512), (75, 512, 192)])
def test_qlora_forward_matches_oracle(rb, orc, M, K, N):
    rng = np.random.default_rng(M * 7 + N)
    w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    x = bf16_round(rng.standard_normal((M, K)))
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    rank = 8
    A = (rng.uniform(-1, 1, size=(rank, K)) / np.sqrt(K)).astype(np.float32)
    B = (rng.standard_normal((N, rank)) * 0.05).astype(np.float32)
    packed, scales = orc.nf4_quantize(w, 64)
    T = rb.Tensor.from_host
    base = rb.QloraLinear(T(w), bias=T(bias))
    got = base.forward(T(x, dtype=_lib.BF16)).to_host()
    want = orc.qlora_forward(x, packed, scales, K, N, 64, bias=bias)
    assert got.shape == (M, N)
    assert rel_l2(got, want) <= 2e-2
    full = rb.QloraLinear(T(w), bias=T(bias), A=T(A), B=T(B), scaling=2.0)
    got = full.forward(T(x.reshape(1, M, K), dtype=_lib.BF16)).to_host()
    want = orc.qlora_forward(x, packed, scales, K, N, 64, bias=bias, A=A, B=B, scaling=2.0)
    assert got.shape == (1, M, N)
    assert rel_l2(got.reshape(M, N), want) <= 2e-2


@pytest.mark.parametrize("M", [1, 2, 4])
def test_small_row_gemv_agrees_with_the_tensor_core_kernel(rb, orc, M):
    """Option nf4_gemv=cuda streams the codes of steps of up to four rows through the CUDA cores (fp16 level
    pairs x fp16 activation-times-scale pairs, block sums in f32) instead of the tensor-core kernel (bf16 level x
    bf16 scale).  Both hold the oracle's tolerance and agree with each other well inside it."""
    rng = np.random.default_rng(M)
    K, N = 2048, 1536
    w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    x = bf16_round(rng.standard_normal((M, K)))
    packed, scales = orc.nf4_quantize(w, 64)
    want = orc.qlora_forward(x, packed, scales, K, N, 64, bias=None)
    T = rb.Tensor.from_host
    layer = rb.QloraLinear(T(w))
    tc = layer.forward(T(x, dtype=_lib.BF16)).to_host()
    rb.set_option("nf4_gemv", "cuda")
    try:
        small = layer.forward(T(x, dtype=_lib.BF16)).to_host()
    finally:
        rb.set_option("nf4_gemv", "tc")
    assert rel_l2(small, want) <= 2e-2 and rel_l2(tc, want) <= 2e-2
    assert rel_l2(small, tc) <= 1e-2


def test_identity_weight_like_the_reference_vector(rb, orc):
    """The reference checks QloraLinear on an identity weight (tests/teager_dispatch.nim:255-262:
    x = [2, 3], bias = [0.5, -1] -> [2.5, 2.0]); the same with the 64-wide blocks this kernel needs."""
    K = N = 64
    w = np.eye(K, dtype=np.float32)
    x = np.zeros((1, K), np.float32)
    x[0, :2] = [2.0, 3.0]
    bias = np.zeros(N, np.float32)
    bias[:2] = [0.5, -1.0]
    layer = rb.QloraLinear(rb.Tensor.from_host(w), bias=rb.Tensor.from_host(bias))
    y = layer.forward(rb.Tensor.from_host(x, dtype=_lib.BF16)).to_host()
    assert np.allclose(y[0, :2], [2.5, 2.0]) and np.all(y[0, 2:] == 0)


def test_shape_errors(rb):
    T = rb.Tensor.from_host
    with pytest.raises(RuntimeError, match="multiples of 64"):
        rb.QloraLinear(T(np.zeros((2, 2), np.float32)))
    layer = rb.QloraLinear(T(np.zeros((64, 64), np.float32)))
    with pytest.raises(RuntimeError, match="inFeatures"):
        layer.forward(T(np.zeros((1, 32), np.float32), dtype=_lib.BF16))


def _nf4_reference_tensors(orc, cfg, tensors):
    """What the reference computes with QLoRA-style frozen weights: every decoder-block Linear weight
    replaced by nf4Dequantize(nf4Quantize(w)) (lora.nim:347-349); embedding, norms, biases and lm_head kept."""
    from rew_b200.weights import tensor_specs
    out = []
    for (name, _), a in zip(tensor_specs(cfg), tensors):
        quantised = a.ndim == 2 and ".layers." in name and name.endswith(".weight")
        out.append(orc.nf4_roundtrip(a, 64) if quantised else a)
    return out


@pytest.mark.parametrize("B,S", [(1, 5), (4, 9), (32, 16), (3, 70)])
def test_nf4_model_logits_match_reference_semantics(rb, orc, B, S):
    """A decoder whose block Linears hold NF4 codes on the device: prefill (codes expanded into a bf16
    scratch, dense tcgen05 Linear) and cached decode (codes dequantised inside the GEMV) against f32
    oracle math on the dequantised weights, rel-L2 <= 2e-2."""
    from rew_b200 import weights as W
    cfg = W.ModelConfig(vocab=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64, ffn=704, max_seq=256,
                        theta=500000.0, dtype=_lib.BF16, mask_kind=1, weight_quant=1)
    t = [orc.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(cfg, seed=4, std=0.05, trivial_affine=False)]
    ref_t = _nf4_reference_tensors(orc, cfg, t)
    prompt = np.random.default_rng(B).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)
    model = rb.CausalLM(cfg).load(t)
    dense = W.ModelConfig(**{**cfg.__dict__, "weight_quant": 0})
    assert model.weight_bytes() < 0.6 * rb.CausalLM(dense).load(t).weight_bytes()
    sess = model.session(B, S + 8)
    nxt, logits = sess.forward(prompt, want_logits=True)
    want = orc.model_forward(cfg, ref_t, prompt, 0, True)[:, -1]
    assert rel_l2(logits, want) <= 2e-2
    ids, last = sess.decode(3, want_logits=True)
    seq = np.concatenate([prompt, nxt[:, None], ids[:, :2]], 1)
    want = orc.model_forward(cfg, ref_t, seq, 0, True)[:, -1]
    assert rel_l2(last, want) <= 2e-2
    # and the quantisation is not a no-op: the unquantised weights give visibly different logits
    assert rel_l2(orc.model_forward(cfg, t, seq, 0, True)[:, -1], want) > 2e-2
