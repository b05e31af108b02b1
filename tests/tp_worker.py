"""One tensor-parallel rank of tests/test_gpu_tp.py (run as a child process, one per GPU)."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, idfile, outfile = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    from rew_b200 import _lib, api, weights as W
    print("rank", rank, "starting", flush=True)
    _lib.init(rank)
    if rank == 0:
        uid = api.comm_unique_id()
        with open(idfile + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(idfile + ".tmp", idfile)
    else:
        t0 = time.time()
        while not os.path.exists(idfile):
            if time.time() - t0 > 60:
                raise RuntimeError("rank 0 never published the communicator id")
            time.sleep(0.05)
        uid = open(idfile, "rb").read()
    api.comm_init(uid, rank, world)
    print("rank", rank, "communicator ready", flush=True)
    fused = len(sys.argv) > 5 and sys.argv[5] in ("fused", "fused_two")
    if fused and sys.argv[5] == "fused_two":
        api.set_option("tp_exchange", "two")   # the two-hop form of the fused exchange
    if fused:  # exchange the IPC handles of the all-reduce heaps through files
        mine = api.comm_peer_alloc(1 << 20, 8 << 20)
        with open("%s.h%d.tmp" % (idfile, rank), "wb") as f:
            f.write(mine)
        os.replace("%s.h%d.tmp" % (idfile, rank), "%s.h%d" % (idfile, rank))
        handles = []
        for r in range(world):
            t0 = time.time()
            while not os.path.exists("%s.h%d" % (idfile, r)):
                if time.time() - t0 > 60:
                    raise RuntimeError("rank %d never published its heap handle" % r)
                time.sleep(0.05)
            handles.append(open("%s.h%d" % (idfile, r), "rb").read())
        api.comm_peer_attach(handles)
        print("rank", rank, "peer heap attached", flush=True)
    results = {}
    for name, dtype, hd, nh, kvh in (("f32", _lib.F32, 32, 8, 2), ("bf16", _lib.BF16, 64, 4, 2)):
        cfg = W.ModelConfig(vocab=512, d_model=256, n_layers=2, n_heads=nh, n_kv_heads=kvh, head_dim=hd, ffn=688, max_seq=128,
                            theta=500000.0, dtype=dtype, mask_kind=1, norm_kind=0, tp_rank=rank, tp_size=world)
        full = W.ModelConfig(**{**cfg.__dict__, "tp_rank": 0, "tp_size": 1})
        t = W.init_weights(full, seed=9, std=0.05, trivial_affine=False)
        if dtype == _lib.BF16:
            t = [W.bf16_round(a) if a.ndim == 2 else a for a in t]
        if name == "f32":
            model = api.CausalLM(cfg).load(t)          # full tensors in, the library cuts out this rank's blocks
        else:
            # shard -> rank: only this rank's block of every tensor crosses the interface (shardLayout's block rule)
            def block(i, tname, g, l, o):
                return t[i][tuple(slice(a, a + n) for a, n in zip(o, l))]
            model = api.CausalLM(cfg)
            g, l, o, pdim = model.tensor_layout(3)     # layer 0 qProj.weight: column-parallel
            assert pdim == 1 and l == (g[0], g[1] // world) and o == (0, rank * g[1] // world), (g, l, o, pdim)
            g, l, o, pdim = model.tensor_layout(9)     # layer 0 outProj.weight: row-parallel
            assert pdim == 0 and l == (g[0] // world, g[1]) and o == (rank * g[0] // world, 0), (g, l, o, pdim)
            if world > 1:  # a block at another rank's offsets is refused
                import ctypes as C
                wrong = np.zeros(l, np.float32)
                off = [((rank + 1) % world) * l[0], 0]
                st = _lib.lib().rewb200_model_set_tensor_shard(model._h, 9, wrong.ctypes.data_as(_lib.F32P), (C.c_int64 * 2)(*l),
                                                               (C.c_int64 * 2)(*off), 2)
                assert st != 0 and b"this rank holds" in _lib.lib().rewb200_last_error()
            model.free()
            model = api.CausalLM(cfg).load_shards(block)
        # 60 prompt rows: every all-reduce of the step is the fused one-shot exchange.  120 rows: the prefill is
        # summed by the two-shot exchange over the heap ("_long"), or through NCCL ("_long_nccl": bf16 payload on the
        # bf16 model); the decode steps behind both are fused again
        for tag, plen, how in (("", 20, "heap"), ("_long", 40, "heap"), ("_long_nccl", 40, "nccl")):
            api.set_option("tp_allreduce", how)
            prompt = np.random.default_rng(3).integers(0, cfg.vocab, size=(3, plen)).astype(np.int32)
            sess = model.session(3, 64)
            ids, logits = sess.generate(prompt, 6, want_logits=True)
            print("rank", rank, name + tag, "done", flush=True)
            results[name + tag + "_ids"] = ids
            results[name + tag + "_logits"] = logits
            sess.free()  # the captured decode graph holds the communicator; release it before comm_destroy
        api.set_option("tp_allreduce", "heap")
    # one decoder layer at the width of the 8B shape (d_model 4096, 32 / 8 heads of 128, FFN 14336): the exchange
    # slots, the split-K policies and the tiles of the real shards; rank 0 also runs the unsharded model
    wide = dict(vocab=2048, d_model=4096, n_layers=1, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, max_seq=128,
                theta=500000.0, dtype=_lib.BF16, mask_kind=1, norm_kind=0)
    full = W.ModelConfig(**wide)
    t = [W.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(full, seed=12, std=0.02, trivial_affine=False)]
    model = api.CausalLM(W.ModelConfig(**wide, tp_rank=rank, tp_size=world)).load(t)
    ref = api.CausalLM(full).load(t) if rank == 0 else None
    for tag, plen in (("", 15), ("_long", 40)):
        prompt = np.random.default_rng(4).integers(0, 2048, size=(4, plen)).astype(np.int32)
        sess = model.session(4, 64)
        ids, logits = sess.generate(prompt, 5, want_logits=True)
        sess.free()
        results["wide" + tag + "_ids"], results["wide" + tag + "_logits"] = ids, logits
        if ref is not None:
            rs = ref.session(4, 64)
            rids, rlogits = rs.generate(prompt, 5, want_logits=True)
            rs.free()
            results["wide" + tag + "_ref_ids"], results["wide" + tag + "_ref_logits"] = rids, rlogits
        print("rank", rank, "wide" + tag, "done", flush=True)
    model.free()
    if ref is not None:
        ref.free()
    np.savez(outfile, **results)
    api.comm_destroy()


if __name__ == "__main__":
    main()
