"""Reading and writing rew checkpoints for the causal-LM models.

Format (Runtime.save / Runtime.load, src/rew/train/runtime.nim:279-364): a directory with
`manifest.json` = {"tensors": [...], "leaf_count": n} and one `tensor_<i>.npy` per pytree leaf, or, for
a sharded leaf, `tensor_<i>_shard_<k>.npy` files with the shard's shape and global offsets.  `.npy`
files are version 1.0, little-endian, C order (src/rew/serialize.nim:261-291); bfloat16 cannot be
stored (serialize.nim:58-60), so parameters are float32.

Leaves are numbered in treeFlatten order (src/rew/pytree.nim:169-199): fields in declaration order,
Param and Buffer leaves alike.  For LlamaForCausalLM (src/rew/models/llama.nim:27-44) that is
  model.embedTokens.weight,
  per layer: selfAttn.{qProj,kProj,vProj,outProj}.{weight,bias}, selfAttn.rope.{cosCached,sinCached},
             mlp.{gateProj,upProj,downProj}.{weight,bias}, inputLayernorm.{gamma,beta},
             postAttentionLayernorm.{gamma,beta},
  model.norm.{gamma,beta}, lmHead.{weight,bias};
for DeepSeekForCausalLM (src/rew/models/deepseek.nim:36-63) the block after the attention is
  moe.gate.{weight,bias}, moe.sharedExperts[*], moe.routedExperts[*] (gateProj, upProj, downProj each),
and lmHead follows norm directly.  The RoPE table buffers are read past: the library rebuilds them
exactly as initRotaryPositionEncoding does.
"""
import json
import os

import numpy as np

from .weights import tensor_specs

ROPE_COS, ROPE_SIN = "<rope.cosCached>", "<rope.sinCached>"


def pytree_leaves(cfg):
    """Names of the checkpoint's leaves in treeFlatten order; canonical tensor names or ROPE_*."""
    out = ["model.embedTokens.weight"]

    def lin(p):
        return [p + ".weight", p + ".bias"]

    def ffn(p):
        return lin(p + ".gateProj") + lin(p + ".upProj") + lin(p + ".downProj")

    for l in range(cfg.n_layers):
        p = "model.layers.%d" % l
        for proj in ("qProj", "kProj", "vProj", "outProj"):
            out += lin(p + ".selfAttn." + proj)
        out += [ROPE_COS, ROPE_SIN]
        if cfg.layer_is_moe(l):
            out += lin(p + ".moe.gate")
            for e in range(cfg.n_shared):
                out += ffn(p + ".moe.sharedExperts.%d" % e)
            for e in range(cfg.n_routed):
                out += ffn(p + ".moe.routedExperts.%d" % e)
        else:
            out += ffn(p + ".mlp")
        out += [p + ".inputLayernorm.gamma", p + ".inputLayernorm.beta",
                p + ".postAttentionLayernorm.gamma", p + ".postAttentionLayernorm.beta"]
    out += ["model.norm.gamma", "model.norm.beta", "lmHead.weight", "lmHead.bias"]
    return out


def rope_tables(head_dim, max_seq, theta):
    """initRotaryPositionEncoding (src/rew/nn/rope.nim:123-138) in numpy float32."""
    i = np.arange(head_dim // 2, dtype=np.float64)
    inv = (np.float32(1.0) / np.power(theta, 2.0 * i / head_dim).astype(np.float32)).astype(np.float32)
    ang = (np.arange(max_seq, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    return np.repeat(np.cos(ang), 2, axis=1).astype(np.float32), np.repeat(np.sin(ang), 2, axis=1).astype(np.float32)


def save_checkpoint(path, cfg, tensors, shard_leaves=None):
    """Writes canonical-order float32 `tensors` as a rew checkpoint.

    shard_leaves: {canonical name: (dim, factor)} writes those leaves as `factor` block shards along
    `dim`, the layout Runtime.save produces for a partitioned leaf (runtime.nim:293-316).
    """
    os.makedirs(path, exist_ok=True)
    by_name = {n: np.ascontiguousarray(t, np.float32) for (n, _), t in zip(tensor_specs(cfg), tensors)}
    cos_t, sin_t = rope_tables(cfg.head_dim, cfg.max_seq, cfg.theta)
    entries = []
    leaves = pytree_leaves(cfg)
    for i, name in enumerate(leaves):
        arr = cos_t if name == ROPE_COS else sin_t if name == ROPE_SIN else by_name[name]
        if shard_leaves and name in shard_leaves:
            dim, factor = shard_leaves[name]
            assert arr.shape[dim] % factor == 0
            local = arr.shape[dim] // factor
            shards = []
            for k in range(factor):
                sl = [slice(None)] * arr.ndim
                sl[dim] = slice(k * local, (k + 1) * local)
                fname = "tensor_%d_shard_%d.npy" % (i, k)
                part = np.ascontiguousarray(arr[tuple(sl)])
                np.save(os.path.join(path, fname), part)
                offs = [0] * arr.ndim
                offs[dim] = k * local
                shards.append({"index": k, "process": 0, "file": fname, "shape": list(part.shape), "offsets": offs})
            entries.append({"index": i, "dtype": "float32", "shape": list(arr.shape), "sharded": True,
                            "sharding_key": "partitioned", "shards": shards})
        else:
            fname = "tensor_%d.npy" % i
            np.save(os.path.join(path, fname), arr)
            entries.append({"index": i, "file": fname, "dtype": "float32", "shape": list(arr.shape), "sharded": False})
    with open(os.path.join(path, "manifest.json"), "w") as f:
        json.dump({"tensors": entries, "leaf_count": len(leaves)}, f)


def load_checkpoint(path, cfg):
    """Reads a rew checkpoint into the canonical tensor list that CausalLM.load takes."""
    with open(os.path.join(path, "manifest.json")) as f:
        manifest = json.load(f)
    leaves = pytree_leaves(cfg)
    if manifest.get("leaf_count") != len(leaves):
        raise ValueError("Runtime.load: checkpoint has %r leaves, this model configuration has %d"
                         % (manifest.get("leaf_count"), len(leaves)))
    want_shape = dict(tensor_specs(cfg))
    found = {}
    for item in manifest["tensors"]:
        idx = item["index"]
        if not 0 <= idx < len(leaves):
            raise ValueError("Runtime.load: leaf index %r out of range" % (idx,))
        name = leaves[idx]
        if name in (ROPE_COS, ROPE_SIN):
            continue
        if item.get("sharded"):
            full = np.empty(tuple(item["shape"]), np.float32)
            seen = np.zeros(full.shape, np.bool_)   # which elements a shard has written
            for sh in item["shards"]:
                part = np.load(os.path.join(path, sh["file"]))
                if list(part.shape) != list(sh["shape"]):
                    raise ValueError("Runtime.load: shard shape %r does not match expected %r" % (part.shape, sh["shape"]))
                offs = list(sh["offsets"])
                if len(offs) != full.ndim or part.ndim != full.ndim or any(
                        o < 0 or o + n > dim for o, n, dim in zip(offs, part.shape, full.shape)):
                    raise ValueError("Runtime.load: shard %r of leaf %d lies outside its shape %r (offsets %r, shape %r)"
                                     % (sh.get("index"), idx, full.shape, offs, part.shape))
                sl = tuple(slice(o, o + n) for o, n in zip(offs, part.shape))
                if seen[sl].any():
                    raise ValueError("Runtime.load: shards of leaf %d overlap (shard %r)" % (idx, sh.get("index")))
                full[sl] = part
                seen[sl] = True
            if not seen.all():
                raise ValueError("Runtime.load: shards of leaf %d do not cover its shape" % idx)
            arr = full
        else:
            arr = np.load(os.path.join(path, item["file"]))
        if arr.dtype != np.float32:
            raise ValueError("Runtime.load: leaf %d (%s) has dtype %s, expected float32" % (idx, name, arr.dtype))
        if tuple(arr.shape) != tuple(want_shape[name]):
            raise ValueError("Runtime.load: leaf %d (%s) has shape %r, expected %r"
                             % (idx, name, tuple(arr.shape), tuple(want_shape[name])))
        found[name] = arr
    missing = [n for n, _ in tensor_specs(cfg) if n not in found]
    if missing:
        raise ValueError("Runtime.load: checkpoint lacks %d tensors, first: %s" % (len(missing), missing[0]))
    return [found[n] for n, _ in tensor_specs(cfg)]


class BlockReader:
    """Reads blocks of a checkpoint's leaves without assembling whole tensors: for a leaf written as shards
    (Runtime.save of a partitioned leaf, src/rew/train/runtime.nim:293-316) only the shard files that overlap
    the requested block are opened, and when the block is exactly one shard (the checkpoint was written with the
    partitioning the model is loaded with) that file is the block.  files_read lists what was opened."""

    def __init__(self, path, cfg):
        self.path = path
        with open(os.path.join(path, "manifest.json")) as f:
            manifest = json.load(f)
        leaves = pytree_leaves(cfg)
        if manifest.get("leaf_count") != len(leaves):
            raise ValueError("Runtime.load: checkpoint has %r leaves, this model configuration has %d"
                             % (manifest.get("leaf_count"), len(leaves)))
        self.want_shape = dict(tensor_specs(cfg))
        self.items = {}
        for item in manifest["tensors"]:
            idx = item["index"]
            if not 0 <= idx < len(leaves):
                raise ValueError("Runtime.load: leaf index %r out of range" % (idx,))
            self.items[leaves[idx]] = item
        self.files_read = []

    def _load(self, fname, mmap=False):
        self.files_read.append(fname)
        return np.load(os.path.join(self.path, fname), mmap_mode="r" if mmap else None)

    def read_block(self, name, local_shape, offsets):
        if name not in self.items:
            raise ValueError("Runtime.load: checkpoint lacks tensor %s" % name)
        item = self.items[name]
        if tuple(item["shape"]) != tuple(self.want_shape[name]):
            raise ValueError("Runtime.load: leaf %s has shape %r, expected %r" % (name, tuple(item["shape"]), tuple(self.want_shape[name])))
        lo = list(offsets)
        hi = [o + n for o, n in zip(offsets, local_shape)]
        sl = tuple(slice(a, b) for a, b in zip(lo, hi))
        if not item.get("sharded"):
            return np.array(self._load(item["file"], mmap=True)[sl], np.float32)
        out = np.empty(tuple(local_shape), np.float32)
        seen = np.zeros(out.shape, np.bool_)
        for sh in item["shards"]:
            s_lo = list(sh["offsets"])
            s_hi = [o + n for o, n in zip(sh["offsets"], sh["shape"])]
            i_lo = [max(a, b) for a, b in zip(lo, s_lo)]
            i_hi = [min(a, b) for a, b in zip(hi, s_hi)]
            if any(a >= b for a, b in zip(i_lo, i_hi)):
                continue                                             # this shard does not touch the block
            part = self._load(sh["file"])
            if list(part.shape) != list(sh["shape"]):
                raise ValueError("Runtime.load: shard shape %r does not match expected %r" % (part.shape, sh["shape"]))
            src = tuple(slice(a - o, b - o) for a, b, o in zip(i_lo, i_hi, s_lo))
            dst = tuple(slice(a - o, b - o) for a, b, o in zip(i_lo, i_hi, lo))
            if seen[dst].any():
                raise ValueError("Runtime.load: shards of leaf %s overlap" % name)
            out[dst] = part[src]
            seen[dst] = True
        if not seen.all():
            raise ValueError("Runtime.load: shards of leaf %s do not cover the requested block" % name)
        return out
