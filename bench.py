"""Headline benchmark: one training step (forward, mean cross-entropy, backward, gradient
all-reduce when data-parallel, AdamW) of the 1.6B-class decoder-only GQA transformer
(28 layers, d_model 2048, 16 query / 4 KV heads, head_dim 128, SwiGLU 5632, vocab 32000,
seq 2048, micro-batch 8 per GPU, bf16 compute, fp32 master weights) on synthetic token ids and
random-init N(0, 0.02) weights.

    python bench.py --gpus N --steps K --warmup W            # this backend (CUDA, sm_100a)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU ops on the host cores
    python bench.py --workload decode [--layers L]           # only the decode workload (batch 32, prompt 512, +256 tokens)

Prints ONE JSON line on rank 0.  For N > 1 launch with torch.distributed.run (one rank per GPU).
`value` is whole-job tokens/s with inputs resident in HBM; `e2e` is the same step driven from
host buffers through the C ABI (pinned H2D of token ids, D2H of the loss, every step).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
PKG = "large-language-model_b200"

MODEL = dict(V=32000, H=2048, I=5632, L=28, nH=16, nKV=4, hd=128, S=2048)
MICRO_BATCH = 8
HYPER = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
METRIC, UNIT = "train_tokens_per_sec", "tokens/s"
# DRAM traffic of the GEMM kernels, average per launch over one training step (ncu dram__bytes_read.sum +
# dram__bytes_write.sum of the 15 GEMM launches of a 1-layer step, the 12 layer GEMMs weighted x28), and the
# algorithmic bytes (each operand read once, the result written once) over the same launches.
GEMM_DRAM_BYTES_PER_LAUNCH = 417951780
GEMM_ALGO_BYTES_PER_LAUNCH = 286487047
GEMM_TRAFFIC_SOURCE = "profiles/gemm_dram_traffic_train_step.md (ncu, 1-layer step scaled by launch counts to 28 layers)"


def model_flops_per_token(m=MODEL):
    """Algorithmic FLOPs of one training step per token: 3 x (projection GEMMs + vocab GEMM) and
    causal attention forward + 2.5x backward (recompute not counted)."""
    q, kv = m["nH"] * m["hd"], m["nKV"] * m["hd"]
    per_layer_gemm = 2 * (m["H"] * (q + 2 * kv) + q * m["H"] + 3 * m["H"] * m["I"])
    attn = 3.5 * (4 * m["nH"] * m["hd"] * m["S"] / 2)       # fwd 4*nH*hd*S/2 per token, bwd 2.5x
    return m["L"] * (3 * per_layer_gemm + attn) + 3 * 2 * m["H"] * m["V"]


def n_params(m=MODEL):
    q, kv = m["nH"] * m["hd"], m["nKV"] * m["hd"]
    return m["L"] * (m["H"] * (q + 2 * kv) + q * m["H"] + 3 * m["H"] * m["I"]) + 2 * m["V"] * m["H"] + m["H"]


DECODE = dict(batch=32, prompt=512, new_tokens=256)


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
    return 6650.0, "fallback (6.65 TB/s)"


def decode_metrics(ctx, bridge, synth, layers=MODEL["L"], reps=2):
    """Autoregressive decode of the same model: batch 32, prompt 512, 256 new tokens, sampling with
    temperature 0.8 / top-p 0.9 / repetition penalty 1.1 (python/pipeline/inference/sampler.py defaults), through
    the host-buffer entry point b200_model_generate.  HBM-bound: per token-step every projection weight is read
    once (bf16) and the K/V cache of every layer is read once for all query heads of a KV head."""
    B, P, NEW = DECODE["batch"], DECODE["prompt"], DECODE["new_tokens"]
    m = dict(MODEL); m["L"] = layers
    shape = bridge.Shape(B=B, S=P + NEW, H=m["H"], I=m["I"], nH=m["nH"], nKV=m["nKV"], hd=m["hd"], V=m["V"], L=layers)
    model = bridge.Model(ctx, shape, "bf16", with_optimizer=False)
    model.init_synthetic(1234, 0.02)
    prompt = synth.token_ids(7, "prompt", (B, P), m["V"])
    cfg = bridge.SamplerConfig.make(temperature=0.8, top_p=0.9, repetition_penalty=1.1, top_k=0, seed=5, whitespace_ids=(220, 256, 198))
    n0 = ctx.launch_count()
    for _ in range(reps):
        t0 = time.perf_counter()
        out, prefill_ms, decode_ms = model.generate(prompt, NEW, cfg)
        wall = time.perf_counter() - t0
    launches = (ctx.launch_count() - n0) // reps
    model.close()
    steps = NEW - 1
    q, kv = m["nH"] * m["hd"], m["nKV"] * m["hd"]
    w_bytes = 2 * (layers * (m["H"] * (q + 2 * kv) + q * m["H"] + 3 * m["H"] * m["I"]) + m["H"] * m["V"])
    t_avg = P + (NEW + 1) / 2.0                       # keys read per step, averaged over the generated positions
    kv_bytes = 2 * layers * B * t_avg * kv * 2
    step_s = decode_ms / 1e3 / steps
    peak, src = hbm_peak()
    achieved = (w_bytes + kv_bytes) / step_s / 1e9
    return {"workload": f"decode: batch {B}, prompt {P}, +{NEW} tokens, {layers}L, KV cache, temperature 0.8 top-p 0.9 rep 1.1",
            "decode_tokens_per_sec": B * steps / (decode_ms / 1e3), "ms_per_token_step": step_s * 1e3,
            "prefill_tokens_per_sec": B * P / (prefill_ms / 1e3), "prefill_ms": prefill_ms,
            "e2e_tokens_per_sec": B * NEW / wall, "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": src, "bytes_per_step": {"weights": w_bytes, "kv_cache_avg": kv_bytes}},
            "distinct_ids": int(len(np.unique(out)))}


def run_decode(args):
    bridge = importlib.import_module(PKG + ".bridge")
    synth = importlib.import_module(PKG + ".synth")
    ctx = bridge.Context(int(os.environ.get("LOCAL_RANK", "0")))
    d = decode_metrics(ctx, bridge, synth, args.layers, reps=max(1, args.steps if args.steps < 3 else 2))
    ctx.close()
    print(json.dumps({"metric": "decode_tokens_per_sec", "value": d["decode_tokens_per_sec"], "unit": UNIT, "n_gpus": 1,
                      "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "config": {"workload": d["workload"]},
                      "decode": d}))


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json, sustained bf16)"
    return 1400.0, "fallback (1.4 PFLOP/s sustained)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(seconds_hint=20.0):
    """The reference's CPU path on this box's host cores, on a bounded sample of the same workload:
    one decoder layer forward+backward and the vocab projection + cross-entropy forward+backward at
    the benchmark's layer shapes on a [1, T] token slice, extrapolated to 28 layers (the reference's
    own per-op ledger method, cpp/tests/bench_blocks.cpp:43-70).  tokens/s = T / (L*t_layer + t_head)."""
    from oracle import oracle
    synth = importlib.import_module(PKG + ".synth")
    use_ref = oracle.have_ref()
    orc = oracle.load_ref() if use_ref else oracle.Oracle()
    T = 128
    cfg = oracle.Config(B=1, S=T, H=MODEL["H"], I=MODEL["I"], nH=MODEL["nH"], nKV=MODEL["nKV"], hd=MODEL["hd"], V=MODEL["V"], L=1)
    lp = synth.layer_params(1, cfg)
    x = synth.normal(1, "x", (1, T, cfg.H))
    g = synth.normal(1, "g", (1, T, cfg.H))
    wout = synth.normal(1, "wout", (cfg.H, cfg.V), 0.02)
    tg = synth.token_ids(1, "tg", (T,), cfg.V)
    t0 = time.perf_counter()
    orc.layer_forward(cfg, x, lp)
    orc.layer_backward(cfg, g, x, lp)
    t_layer = time.perf_counter() - t0
    t0 = time.perf_counter()
    xf = x.reshape(T, cfg.H)
    logits = orc.gemm(xf, wout, T, cfg.V, cfg.H)
    _, dl = orc.cross_entropy(logits, tg)
    orc.gemm(xf, dl, cfg.H, cfg.V, T, transA=True)
    orc.gemm(dl, wout, T, cfg.H, cfg.V, transB=True)
    t_head = time.perf_counter() - t0
    tok_s = T / (MODEL["L"] * t_layer + t_head)
    cores = os.cpu_count() or 1
    return {"value": tok_s, "unit": UNIT, "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"1 decoder layer fwd+bwd ({t_layer:.2f} s) + vocab/CE fwd+bwd ({t_head:.2f} s) on {T} tokens at the "
                      f"benchmark's layer shapes (seq {T}, not 2048), fp32, OpenMP over {cores} threads; extrapolated x{MODEL['L']} layers"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    for i in range(args.warmup + args.steps):
        cb = cpu_baseline()
        if i >= args.warmup:
            vals.append(cb)
    v = float(np.mean([c["value"] for c in vals]))
    cb = vals[-1]
    cb["value"] = v
    T = 128
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * MICRO_BATCH * MODEL["S"] / v, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": workload_name(), "note": "CPU path, bounded sample"},
        "cpu_baseline": cb, "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def workload_name():
    return ("train_step_1p39B_gqa_decoder: 28L d2048 16q/4kv hd128 ffn5632 vocab32000 seq2048 mb8/gpu bf16 "
            "fp32-master AdamW(3e-4,0.9/0.95,wd0.1)")


def run_b200(args):
    import torch
    import torch.distributed as dist
    bridge = importlib.import_module(PKG + ".bridge")
    synth = importlib.import_module(PKG + ".synth")

    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)   # control plane only; gradients go over NCCL
    torch.cuda.set_device(local)
    B, S = args.batch, args.seq
    mcfg = dict(MODEL); mcfg["L"] = args.layers; mcfg["S"] = S
    cfg = bridge.Shape(B=B, S=S, H=mcfg["H"], I=mcfg["I"], nH=mcfg["nH"], nKV=mcfg["nKV"], hd=mcfg["hd"], V=mcfg["V"], L=mcfg["L"])
    ctx = bridge.Context(local)
    model = bridge.Model(ctx, cfg, "bf16", max_batch=B)
    model.init_synthetic(1234, 0.02)            # same weights on every replica
    if world > 1:
        ids = [bridge.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        model.dp_init(ids[0], rank, world)
    tok = synth.token_ids(1000 + rank, "tokens", (B, S + 1), mcfg["V"])
    tokens, targets = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
    d_tok, d_tgt = ctx.array(tokens, "i32"), ctx.array(targets, "i32")
    stream = torch.cuda.ExternalStream(ctx.stream_ptr())

    def barrier():
        ctx.sync()
        if world > 1:
            dist.barrier()

    def step_dev():
        model.train_step(d_tok, d_tgt, B, S, **HYPER)

    for _ in range(args.warmup):
        step_dev()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ctx.profile_gemm(True)
    launches0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step_dev()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = ctx.launch_count() - launches0
    gemm_ms, gemm_flops, gemm_n = ctx.profile_gemm_read()
    ctx.profile_gemm(False)
    loss_dev = float(model._loss.download()[0])
    clocks = sampler.stop() if rank == 0 else None

    # end to end through the host-buffer entry point (pinned H2D of ids, D2H of the loss, each step)
    for _ in range(2):
        model.train_step_host(tokens, targets, **HYPER)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        loss_host = model.train_step_host(tokens, targets, **HYPER)
    ctx.sync()
    e2e_s = time.perf_counter() - t0

    if world > 1:
        t = torch.tensor([ms, e2e_s], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    if rank == 0:
        tokens_total = world * B * S * args.steps
        value = tokens_total / (ms / 1000.0)
        peak, peak_src = measured_peaks()
        achieved = gemm_flops / (gemm_ms / 1000.0) / 1e12 if gemm_ms > 0 else None
        fpt = model_flops_per_token(mcfg)
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name() if (args.layers, B, S) == (MODEL["L"], MICRO_BATCH, MODEL["S"]) else
                       f"REDUCED train step: layers={args.layers} batch={B} seq={S}",
                       "global_batch": world * B, "seq_len": S, "parallelism": f"dp{world}", "params": n_params(mcfg),
                       "l2_policy": "working set per step (>25 GB weights+activations) far exceeds the 126 MB L2"},
            "mfu": {"algorithmic_tflops_per_gpu": fpt * B * S * args.steps / (ms / 1000.0) / 1e12,
                    "six_n_tflops_per_gpu": 6.0 * n_params(mcfg) * B * S * args.steps / (ms / 1000.0) / 1e12,
                    "frac_of_measured_sustained_bf16": fpt * B * S * args.steps / (ms / 1000.0) / 1e12 / peak,
                    "frac_of_nominal_2250": fpt * B * S * args.steps / (ms / 1000.0) / 1e12 / 2250.0},
            "roofline": {"kernel": "gemm_tc2_kernel / gemm_tc_kernel (tcgen05 bf16 GEMM: all projection and vocab GEMMs, fwd + dgrad + wgrad)",
                         "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (achieved / peak) if achieved else None, "peak_source": peak_src,
                         "launches_timed": gemm_n, "share_of_step_time": gemm_ms / ms if ms > 0 else None,
                         "traffic": GEMM_DRAM_BYTES_PER_LAUNCH, "traffic_source": GEMM_TRAFFIC_SOURCE,
                         "algorithmic_bytes_per_launch": GEMM_ALGO_BYTES_PER_LAUNCH},
            "e2e": {"value": tokens_total / e2e_s, "unit": UNIT, "h2d_bytes_per_step": int(2 * B * S * 4),
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches), "clocks": clocks, "loss": {"device_path": loss_dev, "host_path": loss_host},
        }
        if not args.no_cpu_baseline and world == 1:
            out["cpu_baseline"] = cpu_baseline()
    model.close()
    if rank == 0 and world == 1 and not args.no_decode:
        out["decode"] = decode_metrics(ctx, bridge, synth, args.layers)
    if rank == 0:
        print(json.dumps(out))
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL["L"], help="reduced-depth runs are labelled as such (profiling only)")
    ap.add_argument("--batch", type=int, default=MICRO_BATCH)
    ap.add_argument("--seq", type=int, default=MODEL["S"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode workload appended to the 1-GPU line")
    ap.add_argument("--workload", default="train", choices=["train", "decode"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "decode":
        run_decode(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
