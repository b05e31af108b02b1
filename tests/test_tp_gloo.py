"""Host-side check of the tensor-parallel sharding scheme on CPU: two gloo ranks each hold the
column / row / vocabulary slices the engine would upload (block rule of src/rew/sharding.nim:255-270),
run the layer math with the oracle's ops, all-reduce the row-parallel partial sums and all-gather the
vocabulary slices; the result must equal the unsharded oracle forward."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def shard(shape_dim, factor, index):
    """localShape = shape / factor, offset = index * local (sharding.nim:266-270)."""
    assert shape_dim % factor == 0
    local = shape_dim // factor
    return index * local, local


def _worker(rank, world, port, result_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import orc
    from rew_b200 import weights as W
    cfg = W.ModelConfig(vocab=64, d_model=32, n_layers=1, n_heads=4, n_kv_heads=2, head_dim=8, ffn=48, max_seq=32, mask_kind=1)
    t = dict(zip([n for n, _ in W.tensor_specs(cfg)], W.init_weights(cfg, seed=2, std=0.2, trivial_affine=False)))
    ids = np.random.default_rng(0).integers(0, cfg.vocab, size=(2, 7)).astype(np.int32)
    B, S, d, hd = 2, 7, cfg.d_model, cfg.head_dim
    nh_l, kvh_l = cfg.n_heads // world, cfg.n_kv_heads // world
    p = "model.layers.0."

    def col(name, n_full):
        o, n = shard(n_full, world, rank)
        return t[name + ".weight"][:, o:o + n], t[name + ".bias"][o:o + n]

    def row(name, k_full):
        o, n = shard(k_full, world, rank)
        return t[name + ".weight"][o:o + n, :]

    def allreduce(x):
        y = torch.from_numpy(np.ascontiguousarray(x))
        dist.all_reduce(y)
        return y.numpy()

    x = t["model.embedTokens.weight"][ids.ravel()]
    xn = orc.rmsnorm(x, t[p + "inputLayernorm.gamma"], cfg.eps)
    cs, sn = orc.rope_tables(hd, cfg.max_seq, cfg.theta)
    qw, qb = col(p + "selfAttn.qProj", cfg.n_heads * hd)
    kw, kb = col(p + "selfAttn.kProj", cfg.n_kv_heads * hd)
    vw, vb = col(p + "selfAttn.vProj", cfg.n_kv_heads * hd)
    q = orc.linear(xn, qw, qb).reshape(B, S, nh_l, hd).transpose(0, 2, 1, 3)
    k = orc.linear(xn, kw, kb).reshape(B, S, kvh_l, hd).transpose(0, 2, 1, 3)
    v = orc.linear(xn, vw, vb).reshape(B, S, kvh_l, hd).transpose(0, 2, 1, 3)
    a = orc.gqa_attention(orc.rope_apply(q, cs, sn, 0), orc.rope_apply(k, cs, sn, 0), v, True, 1)
    a = a.transpose(0, 2, 1, 3).reshape(B * S, nh_l * hd)
    part = orc.linear(a, row(p + "selfAttn.outProj", cfg.n_heads * hd), np.zeros(d, np.float32))
    x = x + allreduce(part) + t[p + "selfAttn.outProj.bias"]          # bias added once, after the sum
    xn = orc.rmsnorm(x, t[p + "postAttentionLayernorm.gamma"], cfg.eps)
    gw, gb = col(p + "mlp.gateProj", cfg.ffn)
    uw, ub = col(p + "mlp.upProj", cfg.ffn)
    h = orc.silu(orc.linear(xn, gw, gb)) * orc.linear(xn, uw, ub)
    part = orc.linear(h, row(p + "mlp.downProj", cfg.ffn), np.zeros(d, np.float32))
    x = x + allreduce(part) + t[p + "mlp.downProj.bias"]
    xn = orc.rmsnorm(x, t["model.norm.gamma"], cfg.eps)
    lw, lb = col("lmHead", cfg.vocab)
    local = torch.from_numpy(orc.linear(xn, lw, lb))
    gathered = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(gathered, local)
    logits = torch.cat(gathered, 1).numpy().reshape(B, S, cfg.vocab)
    want = orc.model_forward(cfg, list(t.values()), ids, 0, True)
    err = float(np.linalg.norm(logits - want) / np.linalg.norm(want))
    # vocab-parallel greedy: per-rank (max, argmax) then the first-max rule over ranks
    o, n = shard(cfg.vocab, world, rank)
    lv = local.numpy().reshape(B, S, n)[:, -1]
    pair = torch.tensor(np.stack([lv.max(-1), lv.argmax(-1) + o], -1))
    pairs = [torch.empty_like(pair) for _ in range(world)]
    dist.all_gather(pairs, pair)
    allp = torch.stack(pairs, 0).numpy()                     # [world, B, 2]
    best = allp[np.lexsort((allp[..., 1], -allp[..., 0]), axis=0)[0], np.arange(B)]
    greedy_ok = bool(np.array_equal(best[:, 1].astype(np.int64), want[:, -1].argmax(-1)))
    if rank == 0:
        result_q.put((err, greedy_ok))
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_math_matches_unsharded_oracle():
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
    err, greedy_ok = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err < 1e-5
    assert greedy_ok


def test_shard_rule():
    assert shard(28672, 8, 3) == (3 * 3584, 3584)
    assert shard(128256, 8, 7) == (7 * 16032, 16032)
