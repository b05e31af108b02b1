"""Continuous batching over paged KV blocks (PagedKvCache, src/rew/infer/generate.nim:63-88) on the GPU:
requests of different lengths join and leave lanes between decode steps, sharing a small pool of blocks;
every request must produce exactly what the oracle's batch-1 generate() produces for it alone."""
import numpy as np
import pytest

from rew_b200 import weights as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rb():
    from rew_b200 import _lib, api
    _lib.init()
    return api


def _requests(cfg, n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        plen = int(rng.integers(3, 70))
        out.append(dict(id=i, prompt=rng.integers(0, cfg.vocab, size=plen).astype(np.int32), n_new=int(rng.integers(4, 40)),
                        seed=1000 + i))
    return out


def _serve(sess, reqs, lanes, step_sizes):
    """A minimal scheduler: fill idle lanes from the queue, decode a few steps, retire finished requests."""
    pending, active, done, it = list(reqs), {}, {}, 0
    while pending or active:
        for lane in range(lanes):
            if lane not in active and pending:
                r = pending.pop(0)
                r["out"] = [sess.admit(lane, r["prompt"], seed=r["seed"])]
                active[lane] = r
        k = step_sizes[it % len(step_sizes)]
        it += 1
        out = sess.step(k)
        for lane in range(lanes):
            if lane not in active:
                assert np.all(out[lane] == -1)
                continue
            r = active[lane]
            assert sess.lane_length(lane) == len(r["prompt"]) + len(r["out"]) - 1 + k
            r["out"] += out[lane].tolist()
            if len(r["out"]) >= r["n_new"]:
                done[r["id"]] = r["out"][:r["n_new"]]
                sess.release(lane)
                del active[lane]
    return done


@pytest.mark.parametrize("mask_kind", [1, 0])
def test_continuous_batching_matches_per_request_generate(rb, orc, mask_kind):
    cfg = W.tiny_llama(norm_kind=1, mask_kind=mask_kind)
    t = W.init_weights(cfg, seed=21, trivial_affine=False)
    reqs = _requests(cfg, 7, seed=3)
    lanes, blocks = 3, 8                       # 7 usable blocks of 64 tokens for 3 lanes of up to 109 tokens
    sess = rb.CausalLM(cfg).load(t).paged_session(lanes, 112, blocks)
    assert sess.free_blocks() == blocks - 1
    done = _serve(sess, reqs, lanes, step_sizes=[1, 3, 2])
    assert sess.free_blocks() == blocks - 1    # every block came back
    for r in reqs:
        want, _ = orc.generate_greedy(cfg, t, r["prompt"][None, :], r["n_new"])
        assert done[r["id"]] == want[0].tolist(), r["id"]


def test_continuous_batching_with_sampling_matches_oracle(rb, orc):
    cfg = W.tiny_llama(norm_kind=0, mask_kind=1)
    t = W.init_weights(cfg, seed=22)
    reqs = _requests(cfg, 5, seed=4)
    kw = dict(temperature=1.2, top_k=0, top_p=0.9, repetition_penalty=1.15)
    sess = rb.CausalLM(cfg).load(t).paged_session(2, 112, 6)
    sess.set_sampling(**kw)
    done = _serve(sess, reqs, 2, step_sizes=[2, 1])
    for r in reqs:
        want, _ = orc.generate_sampled(cfg, t, r["prompt"][None, :], r["n_new"], seeds=[r["seed"]], **kw)
        assert done[r["id"]] == want[0].tolist(), r["id"]


def test_pool_exhaustion_and_lane_errors(rb):
    cfg = W.tiny_llama(mask_kind=1)
    sess = rb.CausalLM(cfg).load(W.init_weights(cfg, seed=0)).paged_session(2, 128, 3)   # two usable blocks
    p = np.arange(60, dtype=np.int32)
    sess.admit(0, p)
    sess.admit(1, p)
    assert sess.free_blocks() == 0
    with pytest.raises(RuntimeError, match="busy"):
        sess.admit(0, p)
    sess.step(4)                                # 64 tokens each: still one block per lane
    with pytest.raises(RuntimeError, match="out of free blocks"):
        sess.step(1)                            # both lanes would need a second block
    assert sess.lane_length(0) == 64 and sess.lane_length(1) == 64   # nothing moved
    sess.release(1)
    sess.release(1)                             # idempotent
    assert sess.free_blocks() == 1 and sess.lane_length(1) == -1
    out = sess.step(2)                          # lane 0 takes the freed block
    assert np.all(out[1] == -1) and np.all(out[0] >= 0)
    with pytest.raises(RuntimeError, match="out of free blocks"):
        sess.admit(1, p)
    with pytest.raises(RuntimeError, match="out of range"):
        sess.admit(5, p)
    with pytest.raises(RuntimeError, match="paged"):
        sess.generate(p[None, :].repeat(2, 0), 4)
    with pytest.raises(RuntimeError):
        rb.CausalLM(cfg).load(W.init_weights(cfg, seed=0)).paged_session(2, 128, 1)
