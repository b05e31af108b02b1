"""Generates tests/golden/*.npz with the CPU oracle (oracle/rew_oracle.cpp).

The reference (Nim + XLA PJRT plugin) cannot run in the build container, so
these vectors are the oracle's outputs, not the reference's: they pin the
oracle against regressions and travel to the GPU box; model-level parity with
the reference itself stays unpinned.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import orc  # noqa: E402
from rew_b200 import weights as W  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def tiny_generate():
    """The tiny fp32 configuration: tiny Llama, f32, prompt 32 ids (seed 1), 32 greedy tokens."""
    out = {}
    prompt = np.random.default_rng(1).integers(0, 1024, size=(1, 32)).astype(np.int32)
    out["prompt"] = prompt
    for norm_kind, nname in ((0, "rms"), (1, "layernorm")):
        for mask_kind, mname in ((0, "as_written"), (1, "standard")):
            cfg = W.tiny_llama(norm_kind=norm_kind, mask_kind=mask_kind)
            tensors = W.init_weights(cfg, seed=0)
            ids, last, alll = orc.generate_greedy(cfg, tensors, prompt, 32, eos=-1, want_all_logits=True)
            top2 = np.sort(alll[:, 0, :], axis=-1)[:, -2:]
            out["ids_%s_%s" % (nname, mname)] = ids
            out["last_logits_%s_%s" % (nname, mname)] = last
            out["min_margin_%s_%s" % (nname, mname)] = np.float32((top2[:, 1] - top2[:, 0]).min())
    np.savez_compressed(os.path.join(HERE, "tiny_llama_generate.npz"), **out)
    print("tiny_llama_generate.npz", {k: (v.shape if hasattr(v, "shape") else v) for k, v in out.items()})


def small_ops():
    """Small op-level vectors (seeded) for every Tier-B entry point."""
    rng = np.random.default_rng(7)
    out = {}
    x = rng.normal(size=(5, 48)).astype(np.float32)
    w = rng.normal(0, 0.1, size=(48, 40)).astype(np.float32)
    b = rng.normal(0, 0.1, size=(40,)).astype(np.float32)
    g = (1 + rng.normal(0, 0.1, size=(48,))).astype(np.float32)
    be = rng.normal(0, 0.1, size=(48,)).astype(np.float32)
    out.update(lin_x=x, lin_w=w, lin_b=b, lin_y=orc.linear(x, w, b))
    out.update(norm_g=g, norm_b=be, rms_y=orc.rmsnorm(x, g, 1e-5), ln_y=orc.layernorm(x, g, be, 1e-5))
    cs, sn = orc.rope_tables(16, 32, 10000.0)
    xr = rng.normal(size=(2, 3, 4, 16)).astype(np.float32)
    out.update(rope_cos=cs, rope_sin=sn, rope_x=xr, rope_y=orc.rope_apply(xr, cs, sn, offset=5))
    q = rng.normal(size=(2, 4, 6, 16)).astype(np.float32)
    k = rng.normal(size=(2, 2, 6, 16)).astype(np.float32)
    v = rng.normal(size=(2, 2, 6, 16)).astype(np.float32)
    out.update(att_q=q, att_k=k, att_v=v,
               att_plain=orc.gqa_attention(q, k, v, False, 0),
               att_as_written=orc.gqa_attention(q, k, v, True, 0),
               att_standard=orc.gqa_attention(q, k, v, True, 1))
    gw = rng.normal(0, 0.1, size=(48, 24)).astype(np.float32)
    uw = rng.normal(0, 0.1, size=(48, 24)).astype(np.float32)
    dw = rng.normal(0, 0.1, size=(24, 48)).astype(np.float32)
    gb = rng.normal(0, 0.1, size=(24,)).astype(np.float32)
    ub = rng.normal(0, 0.1, size=(24,)).astype(np.float32)
    db = rng.normal(0, 0.1, size=(48,)).astype(np.float32)
    out.update(ffn_gw=gw, ffn_uw=uw, ffn_dw=dw, ffn_gb=gb, ffn_ub=ub, ffn_db=db,
               ffn_y=orc.gated_ffn(x, gw, gb, uw, ub, dw, db))
    rw = rng.normal(0, 0.5, size=(48, 8)).astype(np.float32)
    rb = np.zeros(8, np.float32)
    tw, ti = orc.moe_route(x, rw, rb, 3)
    out.update(route_w=rw, route_b=rb, route_topw=tw, route_topi=ti)
    np.savez_compressed(os.path.join(HERE, "small_ops.npz"), **out)
    print("small_ops.npz", len(out), "arrays")


if __name__ == "__main__":
    orc.build()
    orc.set_accum64(1)
    tiny_generate()
    small_ops()
