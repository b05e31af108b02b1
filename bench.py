#!/usr/bin/env python
"""Decode-throughput benchmark of the rew_b200 backend (one JSON line on stdout).

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--impl reference]

A "step" is one greedy decode step of the whole batch (one token per sequence)
with a KV cache, after a prefill of the prompt.  Workloads (synthetic weights
N(0, 0.02) generated on the device, uniform random prompt ids):

    l8_b32   Llama-3-8B-shaped, bf16, batch 32, prompt 512   (default)
    l8_b1    same model, batch 1
    l8_b128  same model, batch 128, prompt 256 (the 128-row decode tile)
    l70_b16  Llama-3-70B-shaped, bf16, batch 16, prompt 1024; with --gpus N > 1 the model is
             tensor-parallel over the N ranks (heads, FFN columns and vocabulary sharded, NCCL
             all-reduce after o-proj and down-proj): strong scaling
    moe_b64  DeepSeek-V2-Lite-shaped MoE, bf16, global batch 64, prompt 256; with --gpus N > 1 the
             routed experts are sharded over the ranks (expert parallel), every rank owns 64/N
             sequences and each MoE layer does an all-to-all dispatch and combine
With --gpus N > 1 the l8 workloads run N independent replicas (sequences are independent units; no
data-path collective): weak scaling.
    tiny     the tiny fp32 Llama of the parity tests

`value` is decode tokens/s of the whole job with ids, weights and cache resident
in HBM (CUDA events around K graph replays); `e2e` is tokens/s of one generate()
call through the C ABI from host prompt ids to host output ids (prefill, K decode
steps, host<->device copies inside the timed region).  With --impl reference the
reference's CPU path is timed instead: the CPU restatement in oracle/ (the
reference's Nim + XLA-plugin build cannot run here), all host threads.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
SETTLE_S = 0.25            # untimed decode steps run for at least this long after the prefill (see run_model)
SETTLE_MAX_STEPS = 256
E2E_LONG_STEPS = 256       # decode steps of the second end-to-end call (fits the session: max_len has SETTLE_MAX_STEPS of slack)
sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"

WORKLOADS = {
    "l8_b32": dict(model="llama3_8b", batch=32, prompt=512),
    "l8_b1": dict(model="llama3_8b", batch=1, prompt=512),
    "tiny": dict(model="tiny_llama", batch=1, prompt=32),
    "l70_b16": dict(model="llama3_70b", batch=16, prompt=1024, parallel="tp"),
    "l8_b128": dict(model="llama3_8b", batch=128, prompt=256),
    "moe_b64": dict(model="deepseek_v2_lite", batch=64, prompt=256, parallel="ep"),
    # the l8 decoder with its block Linears held as NF4 codes (weight-only, QLoRA's frozen base weights)
    "l8_b32_nf4": dict(model="llama3_8b", batch=32, prompt=512, weight_quant=1),
    "l8_b1_nf4": dict(model="llama3_8b", batch=1, prompt=512, weight_quant=1),
    # one rank's share of the tensor-parallel l70_b16 run as a model of its own (heads, kv heads and FFN width divided by
    # 4 / 8, no exchange): what the sharded kernels cost without the all-reduce, measurable on one GPU
    "l70_tp4shape": dict(model="llama3_70b", batch=16, prompt=1024, shape_div=4),
    "l70_tp8shape": dict(model="llama3_70b", batch=16, prompt=1024, shape_div=8),
    # the attention operator alone: batch 8, 32 query / 8 kv heads, head_dim 128, 4096 positions
    "attn_op": dict(model=None, batch=8, prompt=4096),
}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            j = json.load(f)
        return float(j["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks, power and throttle reasons while the timed region runs.  nvidia-smi needs a
    moment to come up, so it is started ahead of the warm-up steps; every sample carries a timestamp and only
    those inside [mark_begin, mark_end] count.  A region too short to catch two samples (a few decode steps)
    widens to the warm-up steps before it, which run the same launches; `window` says which was used."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap,enforced.power.limit")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.t_warm = self.t0 = self.t1 = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        self.t_warm = time.time()

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            text = open(self.path).read()
            os.unlink(self.path)
        except Exception:
            text = ""
        return self.summarise(text, self.t_warm or 0.0, self.t0 or 0.0, self.t1 or time.time())

    @staticmethod
    def summarise(text, t_warm, t0, t1):
        """Clock record of a run from nvidia-smi's CSV lines (query Q): median SM clock and power over the samples
        whose timestamps fall inside [t0, t1], every throttle reason seen active there."""
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        rows = []
        for line in text.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), float(f[2]), float(f[3]), [v.lower().startswith("active") for v in f[5:9]],
                             f[9] if len(f) > 9 else ""))
            except ValueError:
                continue
        pick = [r for r in rows if t0 <= r[0] <= t1]
        window = "timed region"
        if len(pick) < 2:
            inside = len(pick)
            pick = [r for r in rows if t_warm <= r[0] <= t1]
            window = "warm-up + timed region (the timed region alone caught %d samples)" % inside
        if not pick:
            pick, window = rows, "all samples"
        if pick:
            out["sm_mhz"] = float(np.median([r[1] for r in pick]))
            out["sm_max_mhz"] = float(max(r[2] for r in pick))
            out["power_w"] = float(np.median([r[3] for r in pick]))
            try:
                out["power_limit_w"] = float(pick[0][5])     # read only: the limit this GPU is run under
            except ValueError:
                pass
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            out["reasons"] = sorted({n for r in pick for n, a in zip(names, r[4]) if a})
            out["samples"] = len(pick)
            out["window"] = window
        return out


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def make_cfg(name):
    from rew_b200 import weights as W
    return getattr(W, name)()


def product_config(args, wl, world, model_gb=None):
    """The `config` object of a bench line; both arms print the same one."""
    parallel = "single" if world == 1 else wl.get("parallel", "replicas")
    per_gpu = wl["batch"] // world if parallel == "ep" else wl["batch"]
    cfg = make_cfg(wl["model"])
    return {"workload": args.workload + ("" if args.layers <= 0 else "_%dlayers" % args.layers), "batch_per_gpu": per_gpu,
            "prompt": wl["prompt"], "decode_steps": args.steps, "parallelism": parallel + (str(world) if world > 1 else ""),
            "sampling": args.sampling, "mask": "conventional" if cfg.mask_kind == 1 else "as_written",
            "norm": "rmsNorm" if cfg.norm_kind == 0 else "LayerNorm",
            "l2": "weights streamed per step exceed the 126 MB L2"}


def oracle_sample(args, wl, steps, warm):
    """Times the CPU port on a bounded sample: ONE decoder layer plus the lm_head of the workload's shapes at its
    mean context, every host thread, then extrapolates to all layers by parameter count (both parts are
    weight-streaming GEMMs).  Returns (tokens/s of the full model, seconds per sample step, description, threads)."""
    from oracle import orc
    from rew_b200 import _lib, weights as W
    orc.set_num_threads(os.cpu_count() or 1)   # launchers export OMP_NUM_THREADS=1 for every rank
    cfg = make_cfg(wl["model"])
    full_layers = cfg.n_layers
    cfg.n_layers = 1 if cfg.n_layers > 2 else cfg.n_layers
    cfg.dtype = _lib.F32
    B = wl["batch"]
    ctx = wl["prompt"] + args.warmup + args.steps // 2
    cfg.max_seq = max(cfg.max_seq, ctx + steps + warm + 8)
    rng = np.random.default_rng(0)
    tensors = []
    for name, shape in W.tensor_specs(cfg):
        if len(shape) == 2:
            t = rng.standard_normal(size=shape, dtype=np.float32)
            t *= 0.02
        else:
            t = np.ones(shape, np.float32) if name.endswith("gamma") else np.zeros(shape, np.float32)
        tensors.append(t)
    orc.set_accum64(0)  # f32 accumulation, the fastest setting of the port
    if warm > 0:
        orc.decode_bench(cfg, tensors, B, ctx, warm)
    t = orc.decode_bench(cfg, tensors, B, ctx, steps) / steps
    specs = W.tensor_specs(cfg)
    p_layer = sum(int(np.prod(sh)) for n, sh in specs if ".layers.0." in n and len(sh) == 2)
    p_head = cfg.d_model * cfg.vocab
    layers_run = cfg.n_layers
    p_run = layers_run * p_layer + p_head
    t_full = full_layers * (t * p_layer / p_run) + t * p_head / p_run
    sample = ("%d timed decode steps of %d of %d layers + lm_head, batch %d, context %d, f32, extrapolated by layer count"
              % (steps, layers_run, full_layers, B, ctx))
    return B / t_full, t, t_full, sample, orc.num_threads()


def run_reference(args, wl, rank, world):
    """CPU arm: the oracle port on the host cores, rank 0 only.  Every step is the bounded sample of
    oracle_sample; `ms_per_step` is the time of one sample step, `ms_per_full_step` the extrapolated one."""
    if rank != 0:
        return
    steps = max(1, args.steps)
    warm = max(1, min(args.warmup, 2))
    value, t_sample, t_full, sample, cores = oracle_sample(args, wl, steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t_sample * 1e3, "ms_per_full_step": t_full * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": product_config(args, wl, world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "rew's own CPU path (Nim + XLA PJRT plugin) cannot be built or run here; this is the C++ restatement in oracle/",
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_leg(args, wl):
    """Bounded CPU sample for the GPU arm's line (rank 0, N=1 only)."""
    try:
        value, _, _, sample, cores = oracle_sample(args, wl, 2, 1)
        return {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    except Exception as e:  # the baseline must never take the GPU number down with it
        return {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": "failed: %r" % (e,)}


def run_attention_op(args, rank, local_rank):
    """The attention operator of the decoder alone (bf16, grouped-query, conventional causal mask): a 4096-token
    prefill (tensor roofline) and one decode query over a 4096-entry cache (HBM roofline), device-timed."""
    if rank != 0:
        return
    import ctypes as C
    from rew_b200 import _lib, api
    _lib.init(local_rank)
    for kv in args.option:
        key, _, val = kv.partition("=")
        api.set_option(key, val)
    L = _lib.lib()
    B, nh, kvh, hd, S = 8, 32, 8, 128, args.positions
    rng = np.random.default_rng(0)
    T = api.Tensor.from_host
    k = T(rng.standard_normal((B, kvh, S, hd)).astype(np.float32), dtype=_lib.BF16)
    v = T(rng.standard_normal((B, kvh, S, hd)).astype(np.float32), dtype=_lib.BF16)
    out = {}
    for name, sq in (("prefill", S), ("decode", 1)):
        q = T(rng.standard_normal((B, nh, sq, hd)).astype(np.float32), dtype=_lib.BF16)
        ms, o = C.c_float(), C.c_void_p()
        _lib.check(L.rewb200_gqa_attention_timed(q._h, k._h, v._h, 1 if sq > 1 else 0, 1, max(3, args.steps // 8), C.byref(ms),
                                                 C.byref(o)))
        api.Tensor(o).release()
        q.release()
        out[name] = ms.value
    hbm, which = measured_peaks()
    tf_peak = 1608.7
    pj = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pj):
        with open(pj) as f:
            tf_peak = float(json.load(f).get("bf16_tflops", tf_peak))
    flops = 4.0 * B * nh * hd * S * S / 2          # causal: half of 2 GEMMs of 2*S*S*hd per head
    kv_bytes = 2.0 * B * kvh * S * hd * 2 + 2.0 * B * nh * hd * 2
    tfs = flops / (out["prefill"] * 1e-3) / 1e12
    gbs = kv_bytes / (out["decode"] * 1e-3) / 1e9
    line = {"metric": "attention_op", "value": tfs, "unit": "TFLOP/s (causal prefill)", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": out["prefill"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "attn_op", "batch": B, "q_heads": nh, "kv_heads": kvh, "head_dim": hd, "positions": S,
                       "l2": "K and V (%d MB) %s the 126 MB L2" % (kv_bytes / 1e6, "exceed" if kv_bytes > 126e6 else "fit")},
            "prefill": {"ms": out["prefill"], "tflops": tfs, "frac_of_bf16_peak": tfs / tf_peak, "flops": flops},
            "decode": {"ms": out["decode"], "gbs": gbs, "frac_of_hbm_peak": gbs / hbm, "bytes": kv_bytes},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "traffic": None,
                         "kernel": "attn_decode_kernel<128>", "peak_source": which}}
    print(json.dumps(line), flush=True)


class Comm:
    """Communicator and peer heap of a multi-rank run (one per process), shared by the tensor-parallel and
    expert-parallel measurements."""

    def __init__(self, api, pg, rank, world, allreduce_bytes, alltoall_bytes):
        self.api, self.rank, self.world = api, rank, world
        box = [api.comm_unique_id() if rank == 0 else None]
        pg.broadcast_object_list(box, src=0)
        api.comm_init(box[0], rank, world)
        self.fused = os.environ.get("REW_B200_TP_ALLREDUCE", "fused") == "fused"
        if self.fused:
            mine = api.comm_peer_alloc(allreduce_bytes, alltoall_bytes)
            handles = [None] * world
            pg.all_gather_object(handles, mine)
            api.comm_peer_attach(handles)

    def close(self):
        self.api.comm_destroy()


def a2a_bytes_for(cfg, tokens_per_rank, world):
    """Peer-heap bytes the expert-parallel exchange of one step needs (activations, expert ids, f32 results)."""
    def up(v):
        return (v + 255) // 256 * 256
    slots = tokens_per_rank * cfg.top_k * world
    return up(slots * cfg.d_model * 2) + up(slots * 4) + up(slots * cfg.d_model * 4)


def run_model(args, name, rank, local_rank, world, pg, K, Wm, with_e2e, with_profile):
    """One workload on this process group: prefill, W warm-up steps, K timed decode steps (CUDA events, max over
    ranks), optionally the end-to-end generate() call and the Linear-launch profile.  Returns a dict."""
    import ctypes as C
    from rew_b200 import _lib, api
    L = _lib.lib()
    wl = WORKLOADS[name]
    cfg = make_cfg(wl["model"])
    cfg.weight_quant = wl.get("weight_quant", 0)
    if wl.get("shape_div"):
        dv = wl["shape_div"]
        cfg.n_heads, cfg.n_kv_heads, cfg.ffn = cfg.n_heads // dv, cfg.n_kv_heads // dv, cfg.ffn // dv
        cfg.vocab = cfg.vocab // dv // 8 * 8
    if args.layers > 0:
        cfg.n_layers = args.layers
    B, S = wl["batch"], wl["prompt"]
    max_len = S + Wm + K + 16 + SETTLE_MAX_STEPS
    cfg.max_seq = max(cfg.max_seq, max_len)
    parallel = "single" if world == 1 else wl.get("parallel", "replicas")
    if parallel == "ep":
        cfg.ep_rank, cfg.ep_size = rank, world
        B = B // world
    if parallel == "tp":
        cfg.tp_rank, cfg.tp_size = rank, world
    data_seed = 0 if parallel == "tp" else rank       # tensor-parallel ranks must see the same tokens
    model = api.CausalLM(cfg).init_random(seed=1234 if parallel == "ep" else 1234 + data_seed, std=0.02)
    sess = model.session(B, max_len)
    if args.sampling == "top_k":
        sess.set_sampling(temperature=0.8, top_k=50, repetition_penalty=1.1, seeds=np.arange(B, dtype=np.uint64))
    elif args.sampling == "top_p":
        sess.set_sampling(temperature=0.8, top_k=0, top_p=0.9, repetition_penalty=1.1, seeds=np.arange(B, dtype=np.uint64))
    prompt = np.random.default_rng(1 + data_seed).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)

    # ---- device-resident decode: prefill, W warm-up steps, K timed steps
    # an untimed short prefill first: the first forward of a process loads modules, sets kernel attributes and, on
    # several ranks, makes NCCL connect its peers (hundreds of ms at 8 ranks), none of which is prefill work
    sess.forward(prompt[:, :min(S, 64)])
    sess.reset()
    sess.forward(prompt)
    prefill_ms, _ = sess.last_ms()
    L.rewb200_sync(0, 0)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    def max_over_ranks(v):
        if not pg:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        pg.all_reduce(t, op=pg.ReduceOp.MAX)
        return float(t[0])

    settle = 0
    if Wm > 0:
        sess.decode(Wm)
        # The prefill runs power-capped, and the SM clock stays capped (~1.4 of 1.97 GHz) for about 0.15 s after it:
        # a timed region that starts 20 ms after the prefill measures that transient, not the decode step.  So the
        # untimed part lasts at least SETTLE_S of decode steps; every rank derives the same count from the same
        # max-over-ranks step time (sharded steps contain an exchange, so the ranks must run the same steps).
        step_ms = max_over_ranks(sess.last_ms()[1] / Wm)
        settle = int(min(SETTLE_MAX_STEPS, max(0, math.ceil(args.settle_seconds * 1e3 / max(step_ms, 0.05)) - Wm)))
        if settle > 0:
            sess.decode(settle)
    if pg:
        pg.barrier()
    L.rewb200_sync(0, 0)
    launches0 = L.rewb200_launch_count(0)
    sampler.mark_begin()
    timed_ids = sess.decode(K)
    _, decode_ms = sess.last_ms()
    L.rewb200_sync(0, 0)
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    launches = L.rewb200_launch_count(0) - launches0

    decode_ms = max_over_ranks(decode_ms)
    prefill_ms = max_over_ranks(prefill_ms)
    if pg:
        pg.barrier()
    mult = 1 if parallel == "tp" else world            # B is per rank for replicas and ep
    tokens = B * K * mult
    out = {"name": name, "parallel": parallel, "batch_per_gpu": B, "prompt": S, "value": tokens / (decode_ms * 1e-3),
           "ms_per_step": decode_ms / K, "prefill_ms": prefill_ms, "prefill_tokens_per_s": B * S * mult / (prefill_ms * 1e-3),
           "launches": int(launches), "clocks": clocks, "weight_gb": model.weight_bytes() / 1e9, "cfg": cfg,
           "settle_steps": settle}

    if pg and parallel == "tp":
        # tensor-parallel ranks add the same partials in the same order: the tokens of the timed steps must be the same bits
        import hashlib
        digests = [None] * world
        pg.all_gather_object(digests, hashlib.sha256(np.ascontiguousarray(timed_ids).tobytes()).hexdigest())
        out["ranks_identical"] = len(set(digests)) == 1

    if args.trace:
        # where a step's time goes, per category of launches (events between them: no overlap, so the sum is
        # above the replayed step); max over ranks of the mean of three traced steps
        acc = None
        for _ in range(3):
            t = sess.trace_step()
            acc = t if acc is None else {k: acc[k] + v for k, v in t.items()}
        out["trace_ms"] = {k: round(max_over_ranks(v / 3.0), 4) for k, v in acc.items()}

    # ---- end to end through the C ABI: host prompt ids -> host output ids
    if with_e2e:
        t0 = time.perf_counter()
        ids = sess.generate(prompt, K)
        e2e_s = max_over_ranks(time.perf_counter() - t0)

        out["e2e"] = {"value": tokens / e2e_s, "unit": UNIT, "h2d_bytes_per_step": prompt.nbytes / K,
                      "d2h_bytes_per_step": ids.nbytes / K,
                      "what": "one generate() call: prefill of the prompt + %d decode steps, ids host->device->host" % K}
        if K < E2E_LONG_STEPS:
            # the same call with enough decode steps to show the decode loop's host overhead (with the driver's
            # 20 steps the call is four fifths prefill)
            t0 = time.perf_counter()
            ids = sess.generate(prompt, E2E_LONG_STEPS)
            long_s = max_over_ranks(time.perf_counter() - t0)
            out["e2e_long"] = {"value": B * E2E_LONG_STEPS * mult / long_s, "unit": UNIT, "decode_steps": E2E_LONG_STEPS,
                               "h2d_bytes_per_step": prompt.nbytes / E2E_LONG_STEPS, "d2h_bytes_per_step": ids.nbytes / E2E_LONG_STEPS}

    # ---- rooflines: whole step (weights + KV read once per step per GPU), and the Linear launches alone
    peak, which = measured_peaks()
    kv_bytes = 2 * cfg.n_layers * (cfg.n_kv_heads // cfg.tp_size) * cfg.head_dim * 2 * B * (S + Wm + settle + K / 2.0)
    step_bytes = model.weight_bytes() - cfg.vocab * cfg.d_model * 2 + kv_bytes   # the embedding table is not streamed
    out["step_bytes_per_gpu"] = step_bytes
    out["step_frac"] = step_bytes / (decode_ms / K * 1e-3) / 1e9 / peak
    out["peak"], out["peak_source"] = peak, which
    if with_profile and cfg.n_routed == 0 and cfg.dtype == _lib.BF16:
        ms, nbytes, nl = C.c_float(), C.c_int64(), C.c_int32()
        _lib.check(L.rewb200_session_profile_linears(sess._h, 20, C.byref(ms), C.byref(nbytes), C.byref(nl)))
        out["linear"] = {"ms_per_step": ms.value, "bytes_per_step": nbytes.value, "launches_per_step": nl.value,
                         "gbs": nbytes.value / (ms.value * 1e-3) / 1e9}
    sess.free()
    model.free()
    return out


def sharded_check(rank, world, pg, kind):
    """Correctness of the sharded path inside this run: a small bf16 model split over the ranks against the same
    model unsharded on rank 0 (GPU against GPU; the unsharded path is the one the parity tests hold against the
    oracle).  Returns {"rel_l2": ..., "ids_equal": ...} on rank 0."""
    from rew_b200 import _lib, api, weights as W
    if kind == "tp":
        base = dict(vocab=1024, d_model=512, n_layers=2, n_heads=8, n_kv_heads=8, head_dim=64, ffn=1024, max_seq=128,
                    theta=500000.0, dtype=_lib.BF16, mask_kind=1)
        shard = dict(tp_rank=rank, tp_size=world)
        prompts = {"fused": np.random.default_rng(5).integers(0, 1024, size=(2, 16)).astype(np.int32),
                   "twoshot_prefill": np.random.default_rng(6).integers(0, 1024, size=(4, 24)).astype(np.int32)}
    else:
        base = dict(vocab=512, d_model=256, n_layers=3, n_heads=4, n_kv_heads=4, head_dim=64, ffn=384, max_seq=128,
                    theta=10000.0, eps=1e-6, n_routed=8, n_shared=2, top_k=3, moe_ffn=128, first_dense=384,
                    dtype=_lib.BF16, mask_kind=1)
        shard = dict(ep_rank=rank, ep_size=world)
        prompts = {"peer": np.random.default_rng(7).integers(0, 512, size=(2, 20)).astype(np.int32)}
    full = W.ModelConfig(**base)
    t = [W.bf16_round(a) if a.ndim == 2 else a for a in W.init_weights(full, seed=11, std=0.05, trivial_affine=False)]
    res = {}
    model = api.CausalLM(W.ModelConfig(**base, **shard)).load(t)
    got = {}
    def run(m, pr):
        sess = m.session(pr.shape[0], 64)
        nxt, first = sess.forward(pr, want_logits=True)       # prefill: same input on both sides
        ids, last = sess.decode(4, want_logits=True)           # greedy continuation
        sess.free()
        return nxt, first, ids, last

    for tag, pr in prompts.items():
        got[tag] = run(model, pr)
    model.free()
    if pg:
        pg.barrier()
    if rank == 0:
        ref = api.CausalLM(full).load(t)

        def rel(a, b):
            return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))

        for tag, pr in prompts.items():
            nxt, first, ids, last = run(ref, pr)
            g_nxt, g_first, g_ids, g_last = got[tag]
            same = bool(np.array_equal(nxt, g_nxt) and np.array_equal(ids, g_ids))
            # the last step's logits are comparable only while both greedy paths chose the same tokens
            res[tag] = {"rel_l2_prefill_logits": rel(g_first, first), "ids_equal": same,
                        "rel_l2_last_logits": rel(g_last, last) if same else None}
        ref.free()
    if pg:
        pg.barrier()
    return res


def sub_record(r, which_allreduce=None):
    d = {"workload": r["name"], "parallelism": r["parallel"], "batch_per_gpu": r["batch_per_gpu"], "tokens_per_s": r["value"],
         "ms_per_step": r["ms_per_step"], "prefill_ms": r["prefill_ms"], "prefill_tokens_per_s": r["prefill_tokens_per_s"],
         "per_gpu_step_frac": r["step_frac"], "step_bytes_per_gpu": r["step_bytes_per_gpu"], "gpu_launches": r["launches"],
         "settle_steps": r["settle_steps"], "clocks": r["clocks"]}
    if "linear" in r:
        d["linear_frac"] = r["linear"]["gbs"] / r["peak"]
        d["linear_ms_per_step"] = r["linear"]["ms_per_step"]
    if which_allreduce:
        d["allreduce"] = which_allreduce
    if "ranks_identical" in r:
        d["ranks_identical"] = r["ranks_identical"]
    if "trace_ms" in r:
        d["trace_ms"] = r["trace_ms"]
    return d


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="l8_b32", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="rew_b200", choices=["rew_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-split", action="store_true",
                    help="skip the tensor-parallel (l70_b16) and expert-parallel (moe_b64) sub-records of the default workload")
    ap.add_argument("--option", action="append", default=[], metavar="KEY=VALUE",
                    help="run-time switch passed to rewb200_set_option, e.g. norm=row (repeatable)")
    ap.add_argument("--trace", action="store_true", help="add per-category device times of a decode step to every record")
    ap.add_argument("--settle-seconds", type=float, default=SETTLE_S,
                    help="shortest untimed stretch of decode steps after the prefill (0: only the --warmup steps; profiling aid)")
    ap.add_argument("--positions", type=int, default=4096, help="attn_op only: query / key positions per sequence")
    ap.add_argument("--layers", type=int, default=0, help="profiling aid: keep only this many decoder layers")
    ap.add_argument("--sampling", default="greedy", choices=["greedy", "top_k", "top_p"],
                    help="next-token rule of the decode step; greedy is the metric's configuration")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    rank, local_rank, world = dist_env()

    if args.workload == "attn_op":
        run_attention_op(args, rank, local_rank)
        return
    if args.impl == "reference":
        run_reference(args, wl, rank, world)
        return

    if world > 1 and os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION", "WARN"):
        # keep NCCL's communicator-init lines ("... rank r nranks n ... Init COMPLETE") in the run's log, off stdout
        os.environ["NCCL_DEBUG"] = "INFO"
        os.environ.setdefault("NCCL_DEBUG_SUBSYS", "INIT")
        if "NCCL_DEBUG_FILE" not in os.environ:
            # one file per rank (ranks writing one stream tear each other's lines); echoed to stderr at the end
            os.environ["NCCL_DEBUG_FILE"] = os.path.join(tempfile.gettempdir(), "rew_b200_nccl_%d_%%p.log" % os.getppid())
            os.environ["REW_B200_NCCL_LOG_ECHO"] = "1"

    from rew_b200 import _lib, api, weights as W
    _lib.init(local_rank)
    for kv in args.option:
        k, _, v = kv.partition("=")
        api.set_option(k, v)

    pg = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo")  # host-side rendezvous only: barrier, max over ranks, handle exchange
        pg = dist
    K, Wm = args.steps, args.warmup
    split = args.workload == "l8_b32" and not args.no_split and args.layers <= 0
    parallel = "single" if world == 1 else wl.get("parallel", "replicas")
    comm = None
    if world > 1 and (split or parallel in ("tp", "ep")):
        moe = W.deepseek_v2_lite()
        need_a2a = a2a_bytes_for(moe, (WORKLOADS["moe_b64"]["batch"] // world) * WORKLOADS["moe_b64"]["prompt"], world)
        l70 = WORKLOADS["l70_b16"]
        need_tp = 2 * l70["batch"] * l70["prompt"] * 8192 * 2     # scatter + gather buffer of the two-shot prefill all-reduce
        bulk = max(need_a2a if (split or parallel == "ep") else 0, need_tp if (split or parallel == "tp") else 0)
        comm = Comm(api, pg, rank, world, 64 * 8192 * 4, bulk)   # one-shot slots: 64 rows of d_model 8192 as flagged lines

    r = run_model(args, args.workload, rank, local_rank, world, pg, K, Wm, True, True)
    cfg = r["cfg"]
    peak, which = r["peak"], r["peak_source"]
    if cfg.n_routed > 0 or "linear" not in r:
        ach = r["step_bytes_per_gpu"] / (r["ms_per_step"] * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "frac_nominal": ach / 8000.0,
                    "traffic": None, "kernel": "whole decode step", "bytes_per_step": r["step_bytes_per_gpu"], "peak_source": which}
    else:
        lin = r["linear"]
        kernel = ("nf4_tc_kernel" if cfg.weight_quant else
                  "linear_tc_kernel<32, 0>" if os.environ.get("REW_B200_LINEAR", "tc") != "mma" else "linear_bf16_kernel<32>")
        roofline = {"bound": "hbm", "achieved": lin["gbs"], "peak": peak, "unit": "GB/s", "frac": lin["gbs"] / peak,
                    "frac_nominal": lin["gbs"] / 8000.0,
                    # not measured in this run: DRAM read+write bytes of one profiler capture of the gate|up launch
                    # (239.2 MB for 236.1 MB algorithmic), scaled by the bytes of a step
                    "traffic": None, "traffic_scaled_from_profile": None if cfg.weight_quant else lin["bytes_per_step"] * 1.013,
                    "kernel": kernel, "launches_per_step": lin["launches_per_step"], "ms_per_step": lin["ms_per_step"],
                    "bytes_per_step": lin["bytes_per_step"], "peak_source": which,
                    "step_frac": r["step_frac"], "step_frac_nominal": r["step_frac"] * peak / 8000.0}

    extra = {}
    if split:
        ar = ("fused" if comm and comm.fused else "nccl") if world > 1 else None
        tp = run_model(args, "l70_b16", rank, local_rank, world, pg, K, Wm, False, True)
        extra["tp"] = sub_record(tp, ar)
        ep = run_model(args, "moe_b64", rank, local_rank, world, pg, K, Wm, False, False)
        extra["ep"] = sub_record(ep)
        if world > 1:
            extra["ep"]["exchange"] = "peer_heap" if comm.fused else "nccl"
            extra["tp_check"] = sharded_check(rank, world, pg, "tp")
            extra["ep_check"] = sharded_check(rank, world, pg, "ep")
    if comm:
        comm.close()
    if pg:
        pg.barrier()
        if os.environ.get("REW_B200_NCCL_LOG_ECHO") == "1":
            # the communicator lines of every rank, whole, in rank order
            path = os.environ["NCCL_DEBUG_FILE"].replace("%p", str(os.getpid()))
            for turn in range(world):
                if turn == rank and os.path.exists(path):
                    keep = [l for l in open(path, errors="replace") if "Init COMPLETE" in l or "isAllDirectP2p" in l or "NVLS multicast" in l]
                    sys.stderr.write("".join(keep))
                    sys.stderr.flush()
                    os.unlink(path)
                pg.barrier()
    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wm,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong" if parallel == "tp" else "weak",
        "vs_baseline": None,
        "dtype": ("bf16 activations, NF4 block weights" if cfg.weight_quant else "bf16") if cfg.dtype == _lib.BF16 else "f32",
        "data": "synthetic", "config": product_config(args, wl, world),
        "prefill": {"tokens_per_s": r["prefill_tokens_per_s"], "ms": r["prefill_ms"]},
        "e2e": r["e2e"], "gpu_launches": r["launches"], "clocks": r["clocks"], "roofline": roofline,
    }
    if "e2e_long" in r:
        line["e2e_long"] = r["e2e_long"]
    line["settle"] = ("%d more untimed decode steps after the %d warm-up steps: the SM clock stays capped for ~0.15 s "
                                "after the prefill's power-capped burst, so the untimed part lasts %.2f s" % (r["settle_steps"], Wm, args.settle_seconds))
    if "trace_ms" in r:
        line["trace_ms"] = r["trace_ms"]
    line.update(extra)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_leg(args, wl)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
