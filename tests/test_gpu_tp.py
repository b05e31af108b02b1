"""Tensor parallelism over 2 GPUs (heads / FFN columns / vocabulary sharded, NCCL all-reduce after
o-proj and down-proj) against the single-device oracle.  Needs two GPUs; skipped otherwise."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

from conftest import rel_l2
from rew_b200 import weights as W

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for l in out.splitlines() if l.startswith("GPU "))
    except Exception:
        return 0


def _bundled_nccl():
    import importlib.util
    spec = importlib.util.find_spec("nvidia.nccl")
    if spec and spec.submodule_search_locations:
        p = os.path.join(list(spec.submodule_search_locations)[0], "lib", "libnccl.so.2")
        return p if os.path.exists(p) else None
    return None


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["nccl", "fused", "fused_two"])
def test_tp2_generate_matches_oracle(orc, mode):
    """mode nccl: every all-reduce through NCCL; fused: steps of up to 64 rows use the push all-reduce over
    the peer heap inside the residual+norm kernel (a 60-row prefill too), every rank storing to every peer;
    fused_two: the same with partials sent to the column owner, which returns the sum (option tp_exchange=two); a 120-row prefill is summed by the
    two-shot exchange over the heap and, with option tp_allreduce=nccl, through NCCL (bf16 payload on the bf16
    model)."""
    from rew_b200 import _lib
    with tempfile.TemporaryDirectory() as d:
        idfile = os.path.join(d, "nccl_id")
        env = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
        nccl = _bundled_nccl()
        if nccl and "REW_B200_NCCL" not in env:
            env["REW_B200_NCCL"] = nccl  # the newest NCCL on the machine, without importing its owner
        logs = [open(os.path.join(d, "rank%d.log" % r), "w+") for r in range(2)]
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), "2", idfile,
                                   os.path.join(d, "out%d.npz" % r), mode], env=env, stdout=logs[r], stderr=subprocess.STDOUT)
                 for r in range(2)]
        codes = []
        for p in procs:
            try:
                codes.append(p.wait(timeout=240))
            except subprocess.TimeoutExpired:
                codes.append("timeout")
        for p in procs:
            if p.poll() is None:
                p.kill()  # exactly the children started above
        tails = []
        for f in logs:
            f.seek(0)
            tails.append(f.read()[-3000:])
            f.close()
        assert codes == [0, 0], "rank exit codes %r\n--- rank 0 ---\n%s\n--- rank 1 ---\n%s" % (codes, tails[0], tails[1])
        outs = [np.load(os.path.join(d, "out%d.npz" % r)) for r in range(2)]
    # one layer at the 8B shape's width: ranks bit-identical, and the sharded run against the unsharded one on rank 0
    # (both bf16, different summation orders: far inside the 2e-2 bound; tokens equal up to one near-tie)
    for tag in ("", "_long"):
        assert np.array_equal(outs[0]["wide" + tag + "_ids"], outs[1]["wide" + tag + "_ids"])
        assert np.array_equal(outs[0]["wide" + tag + "_logits"], outs[1]["wide" + tag + "_logits"])
        assert rel_l2(outs[0]["wide" + tag + "_logits"], outs[0]["wide" + tag + "_ref_logits"]) <= 1e-2
        assert (outs[0]["wide" + tag + "_ids"] != outs[0]["wide" + tag + "_ref_ids"]).sum() <= 1
    for name, dtype, hd, nh, kvh in (("f32", _lib.F32, 32, 8, 2), ("bf16", _lib.BF16, 64, 4, 2)):
        cfg = W.ModelConfig(vocab=512, d_model=256, n_layers=2, n_heads=nh, n_kv_heads=kvh, head_dim=hd, ffn=688, max_seq=128,
                            theta=500000.0, dtype=dtype, mask_kind=1, norm_kind=0)
        t = W.init_weights(cfg, seed=9, std=0.05, trivial_affine=False)
        if dtype == _lib.BF16:
            t = [W.bf16_round(a) if a.ndim == 2 else a for a in t]
        for tag, plen in (("", 20), ("_long", 40), ("_long_nccl", 40)):
            prompt = np.random.default_rng(3).integers(0, 512, size=(3, plen)).astype(np.int32)
            key = name + tag
            # both ranks agree bit for bit
            assert np.array_equal(outs[0][key + "_ids"], outs[1][key + "_ids"])
            assert np.array_equal(outs[0][key + "_logits"], outs[1][key + "_logits"])
            if name == "f32":
                want_ids, want_logits = orc.generate_greedy(cfg, t, prompt, 6)
                assert np.array_equal(outs[0][key + "_ids"], want_ids)
                assert rel_l2(outs[0][key + "_logits"], want_logits) <= 1e-5
            else:
                ids = outs[0][key + "_ids"]
                seq = np.concatenate([prompt, ids[:, :5]], 1)
                want = orc.model_forward(cfg, t, seq, 0, True)[:, -1]
                assert rel_l2(outs[0][key + "_logits"], want) <= 2e-2
