"""Host-side check of the expert-parallel scheme on CPU: two gloo ranks each own half of the routed experts
and half of the tokens.  Every (token, expert) pair goes to the owning rank through fixed-capacity per-peer
slot arrays (capacity = local tokens x top_k, meta -1 = empty slot), the owner runs the expert, results come
back in slot order and each token sums its k results in the order j = 0..k-1.  The layer output must equal
the dense all-experts reference math (DeepSeekMoE.forward, src/rew/models/deepseek.nim:122-145)."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def owner(expert, experts_per_rank):
    """Block rule: rank p owns experts [p * E/ep, (p+1) * E/ep)."""
    return expert // experts_per_rank, expert % experts_per_rank


def _exchange(send, world, rank):
    """all-to-all of equal-sized blocks [world, ...] built from all_gather (gloo has no all_to_all on CPU)."""
    t = torch.from_numpy(np.ascontiguousarray(send))
    got = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(got, t)
    return np.stack([g.numpy()[rank] for g in got], 0)       # block p = what rank p addressed to this rank


def _worker(rank, world, port, result_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import orc
    from rew_b200 import weights as W
    cfg = W.ModelConfig(vocab=64, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=8, ffn=48, max_seq=32, mask_kind=1,
                        n_routed=8, n_shared=1, top_k=3, moe_ffn=16, first_dense=48)
    layer = 1
    assert cfg.layer_is_moe(layer)
    tensors = W.init_weights(cfg, seed=6, std=0.3, trivial_affine=False)
    t = dict(zip([n for n, _ in W.tensor_specs(cfg)], tensors))
    p = "model.layers.%d.moe." % layer
    T_all, d, k, E = 12, cfg.d_model, cfg.top_k, cfg.n_routed
    x_all = np.random.default_rng(1).normal(size=(T_all, d)).astype(np.float32)
    T = T_all // world
    x = x_all[rank * T:(rank + 1) * T]
    E_l, cap = E // world, T * k

    def ffn(prefix, rows):
        return orc.gated_ffn(rows, t[prefix + ".gateProj.weight"], t[prefix + ".gateProj.bias"], t[prefix + ".upProj.weight"],
                             t[prefix + ".upProj.bias"], t[prefix + ".downProj.weight"], t[prefix + ".downProj.bias"])

    topw, topi = orc.moe_route(x, t[p + "gate.weight"], t[p + "gate.bias"], k)
    send_x = np.zeros((world, cap, d), np.float32)
    send_meta = np.full((world, cap), -1, np.int32)
    cursor = [0] * world
    pair_slot = np.empty((T, k, 2), np.int64)
    for tok in range(T):
        for j in range(k):
            peer, local_e = owner(int(topi[tok, j]), E_l)
            s = cursor[peer]
            cursor[peer] += 1
            send_x[peer, s], send_meta[peer, s] = x[tok], local_e
            pair_slot[tok, j] = (peer, s)
    assert max(cursor) <= cap
    recv_x, recv_meta = _exchange(send_x, world, rank), _exchange(send_meta, world, rank)
    ret = np.zeros((world, cap, d), np.float32)
    for e in range(E_l):                                      # grouped by local expert, as the grouped GEMM does
        sel = np.argwhere(recv_meta == e)
        if len(sel):
            rows = recv_x[sel[:, 0], sel[:, 1]]
            ret[sel[:, 0], sel[:, 1]] = ffn(p + "routedExperts.%d" % (rank * E_l + e), rows)
    back = _exchange(ret, world, rank)
    out = np.zeros((T, d), np.float32)
    for tok in range(T):
        for j in range(k):
            peer, s = pair_slot[tok, j]
            out[tok] += topw[tok, j] * back[peer, s]
    for e in range(cfg.n_shared):
        out += ffn(p + "sharedExperts.%d" % e, x)
    want = orc.moe_layer(cfg, tensors, layer, x_all)[rank * T:(rank + 1) * T]
    err = float(np.linalg.norm(out - want) / np.linalg.norm(want))
    errs = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(errs, torch.tensor([err], dtype=torch.float64))
    if rank == 0:
        result_q.put([float(e) for e in errs])
    dist.destroy_process_group()


def test_two_rank_expert_parallel_dispatch_matches_dense_reference():
    from oracle import orc
    orc.build()
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    errs = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert max(errs) < 1e-5, errs


def test_owner_rule():
    assert owner(0, 32) == (0, 0) and owner(31, 32) == (0, 31) and owner(32, 32) == (1, 0) and owner(63, 8) == (7, 7)
