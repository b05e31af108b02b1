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
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
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
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["sm_max_mhz"] = float(max(mx))
        out["reasons"] = sorted(reasons)
        return out


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def make_cfg(name):
    from rew_b200 import weights as W
    return getattr(W, name)()


def run_reference(args, wl, rank):
    """CPU arm: the oracle port, timed on the host cores.  Bounded sample: ONE decoder layer plus the
    lm_head of the same shapes at the workload's mean context, extrapolated to all layers."""
    if rank != 0:
        return
    from oracle import orc
    from rew_b200 import _lib, weights as W
    cfg = make_cfg(wl["model"])
    full_layers = cfg.n_layers
    cfg.n_layers = 1 if cfg.n_layers > 2 else cfg.n_layers
    cfg.dtype = _lib.F32
    B = wl["batch"]
    ctx = wl["prompt"] + args.warmup + args.steps // 2
    cfg.max_seq = max(cfg.max_seq, ctx + args.steps + args.warmup + 8)
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
    steps = max(1, min(args.steps, 3))
    warm = max(1, min(args.warmup, 1))
    # lm_head-only time: a model with zero layers is not expressible, so time the 1-layer model and
    # a second call with a doubled step count to separate nothing; instead scale analytically below.
    orc.decode_bench(cfg, tensors, B, ctx, warm)
    t = orc.decode_bench(cfg, tensors, B, ctx, steps) / steps
    # per-step time = layers * t_layer + t_head; split t by parameter count (both are weight-streaming GEMMs)
    specs = W.tensor_specs(cfg)
    p_layer = sum(int(np.prod(s)) for n, s in specs if ".layers.0." in n and len(s) == 2)
    p_head = cfg.d_model * cfg.vocab
    t_layer = t * p_layer / (p_layer + p_head)
    t_head = t * p_head / (p_layer + p_head)
    t_full = full_layers * t_layer + t_head
    value = B / t_full
    sample = ("%d timed decode steps of 1 of %d layers + lm_head, batch %d, context %d, f32, extrapolated by layer count"
              % (steps, full_layers, B, ctx))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t_full * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "batch": B, "prompt": wl["prompt"], "decode_steps": args.steps},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": orc.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "rew's own CPU path (Nim + XLA PJRT plugin) cannot be built or run here; this is the C++ restatement in oracle/",
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_leg(args, wl):
    """Bounded CPU sample for the GPU arm's line (rank 0, N=1 only)."""
    try:
        from oracle import orc
        from rew_b200 import _lib, weights as W
        cfg = make_cfg(wl["model"])
        full_layers = cfg.n_layers
        if cfg.n_layers > 2:
            cfg.n_layers = 1
        cfg.dtype = _lib.F32
        B = wl["batch"]
        ctx = wl["prompt"] + args.steps // 2
        cfg.max_seq = max(cfg.max_seq, ctx + 16)
        rng = np.random.default_rng(0)
        tensors = []
        for name, shape in W.tensor_specs(cfg):
            if len(shape) == 2:
                t = rng.standard_normal(size=shape, dtype=np.float32)
                t *= 0.02
            else:
                t = np.ones(shape, np.float32) if name.endswith("gamma") else np.zeros(shape, np.float32)
            tensors.append(t)
        orc.set_accum64(0)
        orc.decode_bench(cfg, tensors, B, ctx, 1)
        n = 2
        t = orc.decode_bench(cfg, tensors, B, ctx, n) / n
        specs = W.tensor_specs(cfg)
        p_layer = sum(int(np.prod(s)) for nm, s in specs if ".layers.0." in nm and len(s) == 2)
        p_head = cfg.d_model * cfg.vocab
        t_full = full_layers * t * p_layer / (p_layer + p_head) + t * p_head / (p_layer + p_head)
        return {"value": B / t_full, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                "sample": "%d decode steps of 1 of %d layers + lm_head, batch %d, context %d, f32, extrapolated by layer count"
                          % (n, full_layers, B, ctx)}
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
    L = _lib.lib()
    B, nh, kvh, hd, S = 8, 32, 8, 128, 4096
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
                       "l2": "K and V (134 MB) exceed the 126 MB L2"},
            "prefill": {"ms": out["prefill"], "tflops": tfs, "frac_of_bf16_peak": tfs / tf_peak, "flops": flops},
            "decode": {"ms": out["decode"], "gbs": gbs, "frac_of_hbm_peak": gbs / hbm, "bytes": kv_bytes},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "traffic": None,
                         "kernel": "attn_decode_kernel<128>", "peak_source": which}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="l8_b32", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="rew_b200", choices=["rew_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--option", action="append", default=[], metavar="KEY=VALUE",
                    help="run-time switch passed to rewb200_set_option, e.g. norm=row (repeatable)")
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
        run_reference(args, wl, rank)
        return

    import ctypes as C
    from rew_b200 import _lib, api
    _lib.init(local_rank)
    L = _lib.lib()
    for kv in args.option:
        k, _, v = kv.partition("=")
        api.set_option(k, v)

    pg = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo")  # host-side rendezvous only: barrier and max over ranks
        pg = dist

    cfg = make_cfg(wl["model"])
    cfg.weight_quant = wl.get("weight_quant", 0)
    if args.layers > 0:
        cfg.n_layers = args.layers
    B, S, K, Wm = wl["batch"], wl["prompt"], args.steps, args.warmup
    max_len = S + Wm + K + 8
    cfg.max_seq = max(cfg.max_seq, max_len)
    parallel = "single" if world == 1 else wl.get("parallel", "replicas")
    if parallel == "ep":
        cfg.ep_rank, cfg.ep_size = rank, world
        B = B // world
    if parallel in ("tp", "ep"):
        if parallel == "tp":
            cfg.tp_rank, cfg.tp_size = rank, world
        box = [api.comm_unique_id() if rank == 0 else None]
        pg.broadcast_object_list(box, src=0)
        api.comm_init(box[0], rank, world)
        if parallel == "tp" and os.environ.get("REW_B200_TP_ALLREDUCE", "fused") == "fused":
            # decode-size all-reduces run fused into the residual+norm kernel over peer memory
            mine = api.comm_peer_alloc(64 * cfg.d_model * 4)
            handles = [None] * world
            pg.all_gather_object(handles, mine)
            api.comm_peer_attach(handles)
    data_seed = 0 if parallel == "tp" else rank       # tensor-parallel ranks must see the same tokens
    model = api.CausalLM(cfg).init_random(seed=1234 if parallel == "ep" else 1234 + data_seed, std=0.02)
    sess = model.session(B, max_len)
    if args.sampling == "top_k":
        sess.set_sampling(temperature=0.8, top_k=50, repetition_penalty=1.1, seeds=np.arange(B, dtype=np.uint64))
    elif args.sampling == "top_p":
        sess.set_sampling(temperature=0.8, top_k=0, top_p=0.9, repetition_penalty=1.1, seeds=np.arange(B, dtype=np.uint64))
    prompt = np.random.default_rng(1 + data_seed).integers(0, cfg.vocab, size=(B, S)).astype(np.int32)

    # ---- device-resident decode: prefill, W warm-up steps, K timed steps
    sess.forward(prompt)
    prefill_ms, _ = sess.last_ms()
    if Wm > 0:
        sess.decode(Wm)
    if pg:
        pg.barrier()
    L.rewb200_sync(0, 0)
    launches0 = L.rewb200_launch_count(0)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    sess.decode(K)
    _, decode_ms = sess.last_ms()
    L.rewb200_sync(0, 0)
    clocks = sampler.stop() if rank == 0 else None
    launches = L.rewb200_launch_count(0) - launches0
    if pg:
        import torch
        t = torch.tensor([decode_ms], dtype=torch.float64)
        pg.all_reduce(t, op=pg.ReduceOp.MAX)
        decode_ms = float(t[0])
        pg.barrier()
    tokens = B * K * (1 if parallel == "tp" else world)   # B is per rank for replicas and ep
    value = tokens / (decode_ms * 1e-3)

    # ---- end to end through the C ABI: host prompt ids -> host output ids
    t0 = time.perf_counter()
    out = sess.generate(prompt, K)
    e2e_s = time.perf_counter() - t0
    if pg:
        import torch
        t = torch.tensor([e2e_s], dtype=torch.float64)
        pg.all_reduce(t, op=pg.ReduceOp.MAX)
        e2e_s = float(t[0])
    e2e = {"value": tokens / e2e_s, "unit": UNIT, "h2d_bytes_per_step": prompt.nbytes / K,
           "d2h_bytes_per_step": out.nbytes / K,
           "what": "one generate() call: prefill of the prompt + %d decode steps, ids host->device->host" % K}

    # ---- roofline of the dominant kernel (the bf16 weight-streaming Linear)
    roofline = None
    peak, which = measured_peaks()
    kv_b = 2 * cfg.n_layers * (cfg.n_kv_heads // cfg.tp_size) * cfg.head_dim * 2 * B * (S + Wm + K / 2.0)
    if cfg.n_routed > 0:
        # MoE: whole-step figure only (weights of every local expert + KV, read once per step)
        step_bytes = model.weight_bytes() - cfg.vocab * cfg.d_model * 2 + kv_b
        ach = step_bytes / (decode_ms / K * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                    "kernel": "whole decode step", "bytes_per_step": step_bytes, "peak_source": which}
    elif cfg.dtype == _lib.BF16:
        ms = C.c_float()
        nbytes = C.c_int64()
        nl = C.c_int32()
        _lib.check(L.rewb200_session_profile_linears(sess._h, 20, C.byref(ms), C.byref(nbytes), C.byref(nl)))
        peak, which = measured_peaks()
        ach = nbytes.value / (ms.value * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    # dram read+write per step, scaled from the ncu capture of the gate|up launch
                    # (239.2 MB measured for 236.1 MB algorithmic; profiles/linear_tc_kernel_32_decode_l8.md)
                    "traffic": None if cfg.weight_quant else nbytes.value * 1.013,
                    "kernel": ("nf4_tc_kernel" if cfg.weight_quant else "linear_tc_kernel<32, 0>" if os.environ.get("REW_B200_LINEAR", "tc") != "mma" else "linear_bf16_kernel<32>"), "launches_per_step": nl.value, "ms_per_step": ms.value,
                    "bytes_per_step": nbytes.value, "peak_source": which}
        # whole decode step against the same roof: weights + KV read once per step
        kv_bytes = 2 * cfg.n_layers * (cfg.n_kv_heads // cfg.tp_size) * cfg.head_dim * 2 * B * (S + Wm + K / 2.0)
        step_bytes = model.weight_bytes() - cfg.vocab * cfg.d_model * 2 + kv_bytes
        roofline["step_frac"] = step_bytes / (decode_ms / K * 1e-3) / 1e9 / peak

    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wm,
        "ms_per_step": decode_ms / K, "higher_is_better": True, "scaling": "strong" if parallel == "tp" else "weak", "vs_baseline": None,
        "dtype": ("bf16 activations, NF4 block weights" if cfg.weight_quant else "bf16") if cfg.dtype == _lib.BF16 else "f32", "data": "synthetic",
        "config": {"workload": args.workload + ("" if args.layers <= 0 else "_%dlayers" % args.layers), "batch_per_gpu": B, "prompt": S, "decode_steps": K,
                   "parallelism": parallel + (str(world) if world > 1 else ""), "sampling": args.sampling,
                   "l2": "weights per step (%.1f GB) exceed the 126 MB L2" % (model.weight_bytes() / 1e9)},
        "prefill": {"tokens_per_s": B * S * (1 if parallel == "tp" else world) / (prefill_ms * 1e-3), "ms": prefill_ms},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_leg(args, wl)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
