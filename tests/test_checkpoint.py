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


def _hand_written_sharded_checkpoint(path, cfg, t, leaf, shards):
    """A checkpoint written by hand in the layout Runtime.save produces (src/rew/train/runtime.nim:279-321):
    manifest entries with "sharded", "shards": [{"index", "process", "file", "shape", "offsets"}], not by this
    module's own writer.  `shards`: (file index, offsets, array) per shard of canonical tensor `leaf`."""
    os.makedirs(path)
    leaves = CK.pytree_leaves(cfg)
    by_name = dict(zip([n for n, _ in W.tensor_specs(cfg)], t))
    cos_t, sin_t = CK.rope_tables(cfg.head_dim, cfg.max_seq, cfg.theta)
    entries = []
    for i, name in enumerate(leaves):
        arr = cos_t if name == CK.ROPE_COS else sin_t if name == CK.ROPE_SIN else by_name[name]
        if name == leaf:
            recs = []
            for k, offs, part in shards:
                fname = "tensor_%d_shard_%d.npy" % (i, k)
                np.save(os.path.join(path, fname), np.ascontiguousarray(part, np.float32))
                recs.append({"index": k, "process": 0, "file": fname, "shape": list(part.shape), "offsets": list(offs)})
            entries.append({"index": i, "dtype": "float32", "shape": list(arr.shape), "sharded": True,
                            "sharding_key": "partitioned", "shards": recs})
        else:
            np.save(os.path.join(path, "tensor_%d.npy" % i), arr)
            entries.append({"index": i, "file": "tensor_%d.npy" % i, "dtype": "float32", "shape": list(arr.shape), "sharded": False})
    with open(os.path.join(path, "manifest.json"), "w") as f:
        json.dump({"tensors": entries, "leaf_count": len(leaves)}, f)


def test_sharded_leaf_coverage_is_checked(tmp_path):
    """Duplicated, overlapping, missing or out-of-range shards are errors, not uninitialised weights."""
    cfg = W.tiny_llama()
    t = W.init_weights(cfg, seed=3)
    leaf = "model.layers.0.selfAttn.qProj.weight"                     # [256, 256]
    w = dict(zip([n for n, _ in W.tensor_specs(cfg)], t))[leaf]
    halves = [(0, (0, 0), w[:, :128]), (1, (0, 128), w[:, 128:])]
    _hand_written_sharded_checkpoint(str(tmp_path / "ok"), cfg, t, leaf, halves)
    back = CK.load_checkpoint(str(tmp_path / "ok"), cfg)
    assert all(np.array_equal(a, b) for a, b in zip(t, back))
    # the same offsets twice: element counts add up to the full size, the right half is never written
    _hand_written_sharded_checkpoint(str(tmp_path / "dup"), cfg, t, leaf, [(0, (0, 0), w[:, :128]), (1, (0, 0), w[:, :128])])
    with pytest.raises(ValueError, match="overlap"):
        CK.load_checkpoint(str(tmp_path / "dup"), cfg)
    _hand_written_sharded_checkpoint(str(tmp_path / "gap"), cfg, t, leaf, halves[:1])
    with pytest.raises(ValueError, match="do not cover"):
        CK.load_checkpoint(str(tmp_path / "gap"), cfg)
    _hand_written_sharded_checkpoint(str(tmp_path / "oob"), cfg, t, leaf, [halves[0], (1, (0, 200), w[:, 128:])])
    with pytest.raises(ValueError, match="outside its shape"):
        CK.load_checkpoint(str(tmp_path / "oob"), cfg)


def test_block_reader_opens_only_the_shards_a_rank_needs(tmp_path):
    """A leaf saved as 4 column shards: the block of tensor-parallel rank 1 of 4 is one file; of rank 1 of 2
    two files; a row block of a plain leaf comes out of a memory-mapped read."""
    cfg = W.tiny_llama()
    t = W.init_weights(cfg, seed=3, trivial_affine=False)
    by = dict(zip([n for n, _ in W.tensor_specs(cfg)], t))
    q, o = "model.layers.0.selfAttn.qProj.weight", "model.layers.1.selfAttn.outProj.weight"
    CK.save_checkpoint(str(tmp_path / "c"), cfg, t, shard_leaves={q: (1, 4)})
    r = CK.BlockReader(str(tmp_path / "c"), cfg)
    got = r.read_block(q, (256, 64), (0, 64))
    assert np.array_equal(got, by[q][:, 64:128]) and r.files_read == ["tensor_1_shard_1.npy"]
    r.files_read.clear()
    got = r.read_block(q, (256, 128), (0, 128))
    assert np.array_equal(got, by[q][:, 128:]) and r.files_read == ["tensor_1_shard_2.npy", "tensor_1_shard_3.npy"]
    got = r.read_block(o, (128, 256), (128, 0))
    assert np.array_equal(got, by[o][128:])
    with pytest.raises(ValueError, match="lacks tensor"):
        r.read_block("nope", (1,), (0,))


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
