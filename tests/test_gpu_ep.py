"""Expert parallelism over 2 GPUs: routed experts sharded, per-rank sequences, NCCL all-to-all dispatch
and combine in every MoE layer (src/rew/ops/distributed.nim:106-128), against the single-device oracle."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for l in out.splitlines() if l.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_ep2_forward_and_decode_match_oracle(orc):
    import ep_worker
    from test_gpu_tp import _bundled_nccl
    with tempfile.TemporaryDirectory() as d:
        idfile = os.path.join(d, "nccl_id")
        env = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
        nccl = _bundled_nccl()
        if nccl and "REW_B200_NCCL" not in env:
            env["REW_B200_NCCL"] = nccl
        logs = [open(os.path.join(d, "rank%d.log" % r), "w+") for r in range(2)]
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "ep_worker.py"), str(r), "2", idfile,
                                   os.path.join(d, "out%d.npz" % r)], env=env, stdout=logs[r], stderr=subprocess.STDOUT)
                 for r in range(2)]
        codes = []
        for p in procs:
            try:
                codes.append(p.wait(timeout=300))
            except subprocess.TimeoutExpired:
                codes.append("timeout")
        for p in procs:
            if p.poll() is None:
                p.kill()
        tails = []
        for f in logs:
            f.seek(0)
            tails.append(f.read()[-3000:])
            f.close()
        assert codes == [0, 0], "rank exit codes %r\n--- rank 0 ---\n%s\n--- rank 1 ---\n%s" % (codes, tails[0], tails[1])
        outs = [dict(np.load(os.path.join(d, "out%d.npz" % r))) for r in range(2)]
    # one MoE layer at the DeepSeek-V2-Lite width: the expert-parallel ranks against the unsharded model, bit for bit
    for r in range(2):
        assert np.array_equal(outs[r]["wide_ids"], outs[0]["wide_ref_ids%d" % r])
        assert np.array_equal(outs[r]["wide_logits"], outs[0]["wide_ref_logits%d" % r])
    full = ep_worker.config(0, 1)
    t = ep_worker.weights(full)
    for r in range(2):
        prompt = ep_worker.prompt_of(r)
        want = orc.model_forward(full, t, prompt, 0, True)[:, -1]
        assert rel_l2(outs[r]["logits"], want) <= 2e-2
        seq = np.concatenate([prompt, outs[r]["nxt"][:, None], outs[r]["ids"][:, :3]], 1)
        want = orc.model_forward(full, t, seq, 0, True)[:, -1]
        assert rel_l2(outs[r]["last"], want) <= 2e-2
