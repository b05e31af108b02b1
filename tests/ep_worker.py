"""One expert-parallel rank of tests/test_gpu_ep.py (child process, one per GPU): its own sequences,
its own slice of the routed experts, all-to-all dispatch / combine with the other rank."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def config(rank, world):
    from rew_b200 import _lib, weights as W
    return W.ModelConfig(vocab=256, d_model=128, n_layers=3, n_heads=2, n_kv_heads=2, head_dim=64, ffn=192, max_seq=128,
                         theta=10000.0, eps=1e-6, n_routed=8, n_shared=2, top_k=3, moe_ffn=64, first_dense=192,
                         dtype=_lib.BF16, mask_kind=1, ep_rank=rank, ep_size=world)


def weights(cfg):
    from rew_b200 import weights as W
    t = W.init_weights(cfg, seed=31, std=0.08, trivial_affine=False)
    names = [n for n, _ in W.tensor_specs(cfg)]
    for l in (1, 2):  # a router bias that fixes the chosen experts, spread over both ranks' slices
        b = np.zeros(8, np.float32)
        b[[1, 4, 6]] = 50.0
        t[names.index("model.layers.%d.moe.gate.bias" % l)] = b
    return [W.bf16_round(a) if a.ndim == 2 else a for a in t]


def prompt_of(rank):
    return np.random.default_rng(40 + rank).integers(0, 256, size=(2, 19)).astype(np.int32)


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
    # allToAll through the C ABI (src/rew/ops/distributed.nim:106-128): block p of the send buffer lands in block
    # `rank` of rank p's receive buffer
    import ctypes as C
    L = _lib.lib()
    send = api.Tensor.from_host((rank * 100 + np.arange(world, dtype=np.int32))[:, None].repeat(256, 1))
    recv = api.Tensor.from_host(np.full((world, 256), -1, np.int32))
    ptr = lambda t: C.c_void_p(L.rewb200_buffer_device_ptr(t._h))
    _lib.check(L.rewb200_comm_alltoall(0, ptr(send), ptr(recv), 256 * 4))
    got = recv.to_host()
    assert all((got[p] == p * 100 + rank).all() for p in range(world)), got[:, 0]
    # peer heap with an all-to-all region: the default exchange (stores into the owner's memory, counts and
    # flags on the device); handles travel through files like the communicator id
    mine = api.comm_peer_alloc(0, 4 << 20)
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
    cfg = config(rank, world)
    prompt = prompt_of(rank)
    # every rank feeds the same number of tokens per step: the all-to-all slot arrays have one fixed capacity
    sess = api.CausalLM(cfg).load(weights(cfg)).session(prompt.shape[0], 64)
    # The same prompt through the three exchanges must give the same bits: NCCL count-then-prefix (ranks
    # receive 38 and 76 pairs), NCCL fixed capacity, and the peer heap (auto, the default); then the captured
    # decode steps over the peer heap and over NCCL fixed capacity.
    api.set_option("ep_exchange", "prefix")
    nxt, logits = sess.forward(prompt, want_logits=True)
    api.set_option("ep_exchange", "capacity")
    sess.reset()
    nxt2, logits2 = sess.forward(prompt, want_logits=True)
    assert np.array_equal(nxt, nxt2) and np.array_equal(logits, logits2), "prefix and capacity exchange disagree"
    ids2, last2 = sess.decode(4, want_logits=True)
    api.set_option("ep_exchange", "auto")
    sess.reset()
    nxt3, logits3 = sess.forward(prompt, want_logits=True)
    assert np.array_equal(nxt, nxt3) and np.array_equal(logits, logits3), "peer-heap and NCCL exchange disagree (prefill)"
    ids, last = sess.decode(4, want_logits=True)
    assert np.array_equal(ids, ids2) and np.array_equal(last, last2), "peer-heap and NCCL exchange disagree (decode)"
    print("rank", rank, "done", flush=True)
    sess.free()
    # One MoE layer at the DeepSeek-V2-Lite width (d_model 2048, 64 routed experts of width 1408, top-6, two shared
    # experts): 32 experts per rank, real group sizes in the grouped GEMMs and real slot counts in the exchange.
    # Every rank holds the same 8 sequences' worth of weights; rank 0 also runs them unsharded: the expert-parallel
    # run must return the same bits (a token adds its experts' results in fixed order wherever they were computed).
    wide = dict(vocab=1024, d_model=2048, n_layers=2, n_heads=16, n_kv_heads=16, head_dim=128, ffn=2048, max_seq=128,
                theta=10000.0, eps=1e-6, n_routed=64, n_shared=2, top_k=6, moe_ffn=1408, first_dense=2048,
                dtype=_lib.BF16, mask_kind=1)
    full = W.ModelConfig(**wide)
    t = [W.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(full, seed=13, std=0.03, trivial_affine=False)]
    wmodel = api.CausalLM(W.ModelConfig(**wide, ep_rank=rank, ep_size=world)).load(t)
    wprompts = np.random.default_rng(14).integers(0, 1024, size=(world, 8, 40)).astype(np.int32)
    ws = wmodel.session(8, 64)
    wids, wlogits = ws.generate(wprompts[rank], 5, want_logits=True)
    ws.free()
    wmodel.free()
    extra = {}
    if rank == 0:
        ref = api.CausalLM(full).load(t)
        for r in range(world):
            rs = ref.session(8, 64)
            rids, rlogits = rs.generate(wprompts[r], 5, want_logits=True)
            rs.free()
            extra["wide_ref_ids%d" % r], extra["wide_ref_logits%d" % r] = rids, rlogits
        ref.free()
    print("rank", rank, "wide done", flush=True)
    np.savez(outfile, nxt=nxt, logits=logits, ids=ids, last=last, wide_ids=wids, wide_logits=wlogits, **extra)
    api.comm_destroy()


if __name__ == "__main__":
    main()
