"""rew checkpoint directory (manifest.json + tensor_<i>.npy, sharded leaves as tensor_<i>_shard_<k>.npy)
into the canonical tensor list: CPU round trips, and on the GPU a model loaded from a checkpoint."""
import json
import os

import numpy as np
import pytest

from rew_b200 import checkpoint as CK
from rew_b200 import weights as W

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_leaf_order_follows_tree_flatten():
    cfg = W.tiny_llama()
    leaves = CK.pytree_leaves(cfg)
    assert len(leaves) == 1 + 20 * cfg.n_layers + 4
    assert leaves[0] == "model.embedTokens.weight"
    assert leaves[1:9] == ["model.layers.0.selfAttn.%s.%s" % (p, k) for p in ("qProj", "kProj", "vProj", "outProj")
                           for k in ("weight", "bias")]
    assert leaves[9:11] == [CK.ROPE_COS, CK.ROPE_SIN]
    assert leaves[11] == "model.layers.0.mlp.gateProj.weight"
    assert leaves[17:21] == ["model.layers.0.inputLayernorm.gamma", "model.layers.0.inputLayernorm.beta",
                             "model.layers.0.postAttentionLayernorm.gamma", "model.layers.0.postAttentionLayernorm.beta"]
    assert leaves[-4:] == ["model.norm.gamma", "model.norm.beta", "lmHead.weight", "lmHead.bias"]
    moe = W.ModelConfig(vocab=64, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=8, ffn=48, n_routed=4, n_shared=1,
                        top_k=2, moe_ffn=16, first_dense=48)
    ml = CK.pytree_leaves(moe)
    assert len(ml) == 1 + (10 + 6 + 4) + (10 + 2 + 6 * 5 + 4) + 4
    assert set(n for n in ml if not n.startswith("<")) == set(n for n, _ in W.tensor_specs(moe))


def test_round_trip_plain_and_sharded(tmp_path, orc):
    cfg = W.tiny_llama()
    t = W.init_weights(cfg, seed=3, trivial_affine=False)
    CK.save_checkpoint(str(tmp_path / "plain"), cfg, t)
    back = CK.load_checkpoint(str(tmp_path / "plain"), cfg)
    assert all(np.array_equal(a, b) for a, b in zip(t, back))
    man = json.load(open(tmp_path / "plain" / "manifest.json"))
    assert man["leaf_count"] == len(man["tensors"]) == 45
    raw = open(tmp_path / "plain" / "tensor_0.npy", "rb").read(8)
    assert raw[:6] == b"\x93NUMPY" and raw[6:8] == b"\x01\x00"  # .npy v1.0, as serialize.nim writes
    # the RoPE buffers stored in the checkpoint are the reference's tables
    cos_t, sin_t = orc.rope_tables(cfg.head_dim, cfg.max_seq, cfg.theta)
    np.testing.assert_allclose(np.load(tmp_path / "plain" / "tensor_9.npy"), cos_t, atol=1e-6)
    # sharded leaves: column-parallel q, row-parallel o
    shard = {"model.layers.0.selfAttn.qProj.weight": (1, 4), "model.layers.1.selfAttn.outProj.weight": (0, 2)}
    CK.save_checkpoint(str(tmp_path / "sharded"), cfg, t, shard_leaves=shard)
    assert os.path.exists(tmp_path / "sharded" / "tensor_1_shard_3.npy")
    back = CK.load_checkpoint(str(tmp_path / "sharded"), cfg)
    assert all(np.array_equal(a, b) for a, b in zip(t, back))


def test_load_errors(tmp_path):
    cfg = W.tiny_llama()
    t = W.init_weights(cfg, seed=3)
    CK.save_checkpoint(str(tmp_path / "c"), cfg, t)
    other = W.tiny_llama()
    other.n_layers = 3
    with pytest.raises(ValueError, match="leaves"):
        CK.load_checkpoint(str(tmp_path / "c"), other)
    np.save(tmp_path / "c" / "tensor_0.npy", np.zeros((3, 3), np.float32))
    with pytest.raises(ValueError, match="shape"):
        CK.load_checkpoint(str(tmp_path / "c"), cfg)


@pytest.mark.gpu
def test_model_from_checkpoint_generates_the_golden_ids(tmp_path):
    from rew_b200 import _lib, api
    _lib.init()
    z = np.load(os.path.join(GOLD, "tiny_llama_generate.npz"))
    cfg = W.tiny_llama()
    CK.save_checkpoint(str(tmp_path / "c"), cfg, W.init_weights(cfg, seed=0),
                       shard_leaves={"model.layers.0.mlp.gateProj.weight": (1, 2)})
    sess = api.CausalLM(cfg).load(CK.load_checkpoint(str(tmp_path / "c"), cfg)).session(1, 64)
    assert np.array_equal(sess.generate(z["prompt"], 32), z["ids_rms_as_written"])
