"""Headline benchmark: one training step (forward, mean cross-entropy, backward, gradient
all-reduce when data-parallel, AdamW) of the 1.6B-class decoder-only GQA transformer
(28 layers, d_model 2048, 16 query / 4 KV heads, head_dim 128, SwiGLU 5632, vocab 32000,
seq 2048, micro-batch 8 per GPU, bf16 compute, fp32 master weights) on synthetic token ids and
random-init N(0, 0.02) weights.

    python bench.py --gpus N --steps K --warmup W            # this backend (CUDA, sm_100a)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU ops on the host cores
    python bench.py --workload decode [--layers L]           # only the decode workload (batch 32, prompt 512, +256 tokens)

    python bench.py --workload ops                           # only the per-op figures (attention, projections, bandwidth kernels)
    python bench.py --workload trace --steps 3               # in-step device time per launch site (table on stdout, not a JSON line)

Prints ONE JSON line on rank 0.  For N > 1 launch with torch.distributed.run (one rank per GPU).
`value` is whole-job tokens/s with inputs resident in HBM; `e2e` is the same step driven from
host buffers through the C ABI (pinned H2D of token ids, D2H of the loss, every step).
At N = 1 the line also carries `attention` (causal GQA attention op at batch 8, seq 2048, 16/4 heads, head_dim 128:
forward, backward, both in TFLOP/s), `ops` (every projection GEMM of the model at 16384 tokens as forward, data-gradient
and weight-gradient, the vocabulary projection fused with cross-entropy, and the bandwidth-bound kernels in GB/s) and
`decode`.  At N > 1 it carries `dp_check`: replicas end with bit-identical weights, and the data-parallel loss and
gradients of a 2-layer model equal a single-device run on the concatenated batch.
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
GEMM_DRAM_BYTES_PER_LAUNCH = 442382891
GEMM_ALGO_BYTES_PER_LAUNCH = 301730064
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


_ATTN_CPU = {}      # the S = 2048 attention sample is measured once per process and reused


def _omp_all_cores():
    """The CPU arm uses every host core at every N (torch.distributed.run exports OMP_NUM_THREADS=1 to its workers)."""
    n = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(n)
    return n


def cpu_baseline():
    """The reference's CPU path on this box's host cores, as a ledger of bounded samples at the benchmark's shapes
    (the reference's own per-op ledger method, cpp/tests/bench_blocks.cpp:43-70, 861-935):
      t_attn   attention block forward+backward at the FULL sequence length 2048 for one sequence and one KV group
               (4 query heads + 1 KV head of head_dim 128, d_model 512 slice: the reference requires
               n_heads*head_dim == d_model), measured once per process; minus the same block at 128 tokens x16, which
               removes the slice's own projections and leaves the O(S^2) core (cpp/src/Attention.cpp:236-280, 531-540);
      t_layer  one decoder layer forward+backward on 128 tokens at the real layer shapes (projections, SwiGLU, norms:
               everything linear in tokens; its attention core at 128 tokens is 1/256 of the real one per token);
      t_head   vocabulary projection + cross-entropy forward+backward on 128 tokens.
    One sequence of 2048 tokens then costs L * (nKV * t_core + 16 * t_layer) + 16 * t_head."""
    cores = _omp_all_cores()
    from oracle import oracle
    synth = importlib.import_module(PKG + ".synth")
    use_ref = oracle.have_ref()
    orc = oracle.load_ref() if use_ref else oracle.Oracle()
    T, S, G = 128, MODEL["S"], MODEL["nH"] // MODEL["nKV"]
    hd = MODEL["hd"]

    def attn_block(seq):
        c = oracle.Config(B=1, S=seq, H=G * hd, I=8, nH=G, nKV=1, hd=hd, V=8, L=1)
        x, g = synth.normal(2, "ax", (1, seq, c.H)), synth.normal(2, "ag", (1, seq, c.H))
        w = [synth.normal(2, n, shp, 0.02) for n, shp in (("aq", (c.H, G * hd)), ("ak", (c.H, hd)), ("av", (c.H, hd)), ("ao", (G * hd, c.H)))]
        t0 = time.perf_counter()
        orc.attention_layer(c, x, *w, gout=g)
        return time.perf_counter() - t0

    if "t_full" not in _ATTN_CPU:
        _ATTN_CPU["t_full"] = attn_block(S)
    t_small = attn_block(T)
    t_core = max(_ATTN_CPU["t_full"] - (S // T) * t_small, 0.5 * _ATTN_CPU["t_full"])
    cfg = oracle.Config(B=1, S=T, H=MODEL["H"], I=MODEL["I"], nH=MODEL["nH"], nKV=MODEL["nKV"], hd=hd, V=MODEL["V"], L=1)
    if "inputs" not in _ATTN_CPU:       # the seeded inputs are generated once; every step times the same work
        _ATTN_CPU["inputs"] = (synth.layer_params(1, cfg), synth.normal(1, "x", (1, T, cfg.H)), synth.normal(1, "g", (1, T, cfg.H)),
                               synth.normal(1, "wout", (cfg.H, cfg.V), 0.02), synth.token_ids(1, "tg", (T,), cfg.V))
    lp, x, g, wout, tg = _ATTN_CPU["inputs"]
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
    per_seq = MODEL["L"] * (MODEL["nKV"] * t_core + (S // T) * t_layer) + (S // T) * t_head
    return {"value": S / per_seq, "unit": UNIT, "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"ledger at the benchmark's shapes, fp32, OpenMP over {cores} threads: attention core fwd+bwd at seq {S} for one "
                      f"sequence and one KV group ({_ATTN_CPU['t_full']:.1f} s measured once per process, {t_core:.1f} s after removing the "
                      f"slice's projections; x{MODEL['nKV']} groups); one decoder layer fwd+bwd on {T} tokens ({t_layer:.2f} s, x{S // T}); "
                      f"vocab projection + cross-entropy fwd+bwd on {T} tokens ({t_head:.2f} s, x{S // T}); x{MODEL['L']} layers. "
                      "GEMM stand-in for Accelerate's cblas_sgemm: OpenMP row-parallel triple loop (oracle/shim/bridge_cpu_stub.cpp); "
                      "the attention backward is the reference's serial loop over (batch, head, query)",
            "seconds": {"attention_core_one_group_seq2048": t_core, "layer_128_tokens": t_layer, "head_128_tokens": t_head}}


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
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * MICRO_BATCH * MODEL["S"] / v, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": make_config(max(1, args.gpus), MICRO_BATCH, MODEL["S"], MODEL["L"]),
        "note": "CPU path: ms_per_step is the extrapolated time of one full step (8 x 2048 tokens), not the duration of a sample",
        "cpu_baseline": cb, "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def workload_name():
    return ("train_step_1p39B_gqa_decoder: 28L d2048 16q/4kv hd128 ffn5632 vocab32000 seq2048 mb8/gpu bf16 "
            "fp32-master AdamW(3e-4,0.9/0.95,wd0.1)")


def make_config(world, B, S, layers):
    m = dict(MODEL); m["L"] = layers; m["S"] = S
    return {"workload": workload_name() if (layers, B, S) == (MODEL["L"], MICRO_BATCH, MODEL["S"]) else
            f"REDUCED train step: layers={layers} batch={B} seq={S}",
            "global_batch": world * B, "seq_len": S, "parallelism": f"dp{world}", "params": n_params(m),
            "l2_policy": "working set per step (>25 GB weights+activations) far exceeds the 126 MB L2"}


def peaks_all():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"bf16_burst": float(d["bf16_tflops"]), "bf16_sustained": float(d["bf16_tflops_sustained"]), "hbm": float(d["hbm_gbs"]),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class OpTimer:
    """CUDA-event timing of back-to-back launches on the context's stream (device time, after warm-up)."""

    def __init__(self, ctx, torch):
        self.ctx, self.torch = ctx, torch
        self.stream = torch.cuda.ExternalStream(ctx.stream_ptr())

    def ms(self, fn, reps=20, warm=3):
        for _ in range(warm):
            fn()
        e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        self.ctx.sync()
        e0.record(self.stream)
        for _ in range(reps):
            fn()
        e1.record(self.stream)
        self.ctx.sync()
        return e0.elapsed_time(e1) / reps


def _fill(ctx, bridge, arr, seed, std):
    ctx._check(ctx.lib.b200_fill_normal(ctx.h, arr.ptr, arr.code, arr.size, seed, std))
    return arr


ATTN = dict(B=8, S=2048, nH=16, nKV=4, hd=128)


def attention_metrics(ctx, bridge, torch, cpu_check=True, reps=20):
    """Causal GQA attention op, bf16: batch 8, seq 2048, 16 query / 4 KV heads, head_dim 128, Q/K/V/dO ~ N(0,1), through
    b200_flash_attn_fwd and b200_flash_attn_bwd (layouts of the reference call: Q [B,nH,S,hd], K/V [B,nKV,S,hd], O/dO
    [B,S,nH*hd]).  Two input sets alternate between launches (336 MB in flight against the 126 MB L2).
    FLOPs: forward 4*B*nH*S^2*hd/2, backward 2.5x (recomputation not counted).  With cpu_check, one (batch, KV group)
    slice is recomputed by the CPU checker inside the CPU-baseline leg: its time and the GPU's relative error."""
    B, S, nH, nKV, hd = (ATTN[k] for k in ("B", "S", "nH", "nKV", "hd"))
    sets = []
    for i in range(2):
        q = _fill(ctx, bridge, ctx.empty((B, nH, S, hd), "bf16"), 11 + 10 * i, 1.0)
        k = _fill(ctx, bridge, ctx.empty((B, nKV, S, hd), "bf16"), 12 + 10 * i, 1.0)
        v = _fill(ctx, bridge, ctx.empty((B, nKV, S, hd), "bf16"), 13 + 10 * i, 1.0)
        do = _fill(ctx, bridge, ctx.empty((B, S, nH * hd), "bf16"), 14 + 10 * i, 1.0)
        o, lse = ctx.empty((B, S, nH * hd), "bf16"), ctx.empty((B, nH, S), "f32")
        grads = (ctx.empty(q.shape, "bf16"), ctx.empty(k.shape, "bf16"), ctx.empty(v.shape, "bf16"))
        sets.append((q, k, v, do, o, lse, grads))
    lib, h = ctx.lib, ctx.h
    n = [0]

    def fwd():
        q, k, v, do, o, lse, g = sets[n[0] & 1]; n[0] += 1
        ctx._check(lib.b200_flash_attn_fwd(h, q.ptr, k.ptr, v.ptr, o.ptr, lse.ptr, B, nH, nKV, S, hd, bridge.BF16))

    def bwd():
        q, k, v, do, o, lse, g = sets[n[0] & 1]; n[0] += 1
        ctx._check(lib.b200_flash_attn_bwd(h, q.ptr, k.ptr, v.ptr, o.ptr, do.ptr, lse.ptr, g[0].ptr, g[1].ptr, g[2].ptr, B, nH, nKV, S, hd, bridge.BF16))

    t = OpTimer(ctx, torch)
    l0 = ctx.launch_count()
    ms_f = t.ms(fwd, reps)
    fwd(); fwd()                         # both sets hold O and lse of their own inputs before the backward is timed
    ms_b = t.ms(bwd, reps)
    launches = ctx.launch_count() - l0
    f_fwd = 4.0 * B * nH * S * S * hd / 2
    f_bwd = 2.5 * f_fwd
    pk = peaks_all()

    def entry(ms, fl):
        tf = fl / (ms / 1e3) / 1e12
        return {"ms": ms, "tflops": tf, "frac_of_burst": tf / pk["bf16_burst"], "frac_of_sustained": tf / pk["bf16_sustained"]}

    out = {"workload": f"causal GQA attention bf16: batch {B}, seq {S}, {nH}q/{nKV}kv heads, head_dim {hd}",
           "forward": entry(ms_f, f_fwd), "backward": entry(ms_b, f_bwd), "forward_backward": entry(ms_f + ms_b, f_fwd + f_bwd),
           "launches_timed": reps, "gpu_launches": int(launches), "peak_source": pk["source"],
           "l2_policy": "two input sets alternate; 336 MB of operands and results per pair of launches"}
    if cpu_check:
        out["cpu_check"] = attention_cpu_check(ctx, sets[0], B, S, nH, nKV, hd)
    for st in sets:
        for a in st[:6] + st[6]:
            a.free()
    return out


def attention_cpu_check(ctx, st, B, S, nH, nKV, hd, b=5, kvh=2):
    """CPU-baseline leg of the attention op: the CPU checker computes forward and backward for one (batch, KV group)
    slice at the full sequence length on the same bf16 inputs; returns its time and the GPU results' relative errors."""
    _omp_all_cores()
    from oracle import oracle
    q, k, v, do, o, lse, grads = st
    G = nH // nKV
    hs = slice(kvh * G, (kvh + 1) * G)
    Q, K, V, dO = q.download()[b:b + 1, hs], k.download()[b:b + 1, kvh:kvh + 1], v.download()[b:b + 1, kvh:kvh + 1], do.download()
    dO = np.ascontiguousarray(dO[b:b + 1].reshape(1, S, nH, hd)[:, :, hs].reshape(1, S, G * hd))
    orc = oracle.Oracle()
    t0 = time.perf_counter()
    eo = orc.attention_forward(Q, K, V)
    t_f = time.perf_counter() - t0
    t0 = time.perf_counter()
    edq, edk, edv = orc.attention_backward(Q, K, V, dO)
    t_b = time.perf_counter() - t0

    def rel(a, e):
        a, e = np.asarray(a, np.float64).ravel(), np.asarray(e, np.float64).ravel()
        return float(np.linalg.norm(a - e) / (np.linalg.norm(e) + 1e-30))

    go = o.download()[b:b + 1].reshape(1, S, nH, hd)[:, :, hs].reshape(1, S, G * hd)
    # the GPU's dK/dV of this KV head sum over exactly these G query heads, so the slice is self-contained
    r = {"O": rel(go, eo), "dQ": rel(grads[0].download()[b:b + 1, hs], edq), "dK": rel(grads[1].download()[b:b + 1, kvh:kvh + 1], edk),
         "dV": rel(grads[2].download()[b:b + 1, kvh:kvh + 1], edv)}
    fl = 4.0 * G * S * S * hd / 2
    return {"slice": f"batch {b}, KV head {kvh} (query heads {kvh * G}..{kvh * G + G - 1}), seq {S}", "rel_err": r, "tolerance": 2e-2,
            "cpu_seconds": {"forward": t_f, "backward": t_b}, "cpu_gflops": {"forward": fl / t_f / 1e9, "backward": 2.5 * fl / t_b / 1e9},
            "cpu_kind": "port (oracle/block_oracle.c, fp32)", "cores": os.cpu_count()}


def ops_metrics(ctx, bridge, torch, reps=20):
    """Per-op figures at the model's shapes with M = 8 x 2048 = 16384 tokens, bf16: every projection as forward (NN), data
    gradient (NT) and weight gradient (TN, fp32 result) in TFLOP/s; the bandwidth-bound kernels in GB/s over their
    algorithmic bytes (each input read once, each output written once).  Operands are far larger than L2."""
    M, H, I, V = MICRO_BATCH * MODEL["S"], MODEL["H"], MODEL["I"], MODEL["V"]
    Q, KV = MODEL["nH"] * MODEL["hd"], MODEL["nKV"] * MODEL["hd"]
    pk = peaks_all()
    t = OpTimer(ctx, torch)
    lib, h, BF, F32 = ctx.lib, ctx.h, bridge.BF16, bridge.F32
    big_a = _fill(ctx, bridge, ctx.empty((M * V,), "bf16"), 1, 1.0)          # activations / dY, up to [M, V]
    big_c = ctx.empty((M * V,), "bf16")
    w = _fill(ctx, bridge, ctx.empty((H * V,), "bf16"), 2, 0.02)             # weights, up to [H, V]
    c32 = ctx.empty((H * V,), "f32")
    l0 = ctx.launch_count()
    gemms = {}

    def tf_entry(ms, fl):
        tf = fl / (ms / 1e3) / 1e12
        return {"ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_burst": round(tf / pk["bf16_burst"], 3), "frac_of_sustained": round(tf / pk["bf16_sustained"], 3)}

    for name, K, N in (("qkv", H, Q + 2 * KV), ("o", Q, H), ("gate_up", H, 2 * I), ("down", I, H), ("vocab", H, V)):
        fl = 2.0 * M * N * K
        fwd = lambda: ctx._check(lib.b200_gemm(h, big_a.ptr, w.ptr, big_c.ptr, M, N, K, 0, 0, 0, BF, BF))
        if name == "gate_up":          # the engine's form: SwiGLU in the epilogue, gate|up kept for the backward
            act = ctx.empty((M * I,), "bf16")
            fwd = lambda: ctx._check(lib.b200_gemm_ffn(h, big_a.ptr, w.ptr, big_c.ptr, act.ptr, M, I, K, BF))
        dgrad = lambda: ctx._check(lib.b200_gemm(h, big_a.ptr, w.ptr, big_c.ptr, M, K, N, 0, 1, 0, BF, BF))      # dY[M,N] * W[K,N]^T
        wgrad = lambda: ctx._check(lib.b200_gemm(h, big_c.ptr, big_a.ptr, c32.ptr, K, N, M, 1, 0, 0, BF, F32))    # X[M,K]^T * dY[M,N]
        gemms[name] = {"shape": f"[{M},{K}]x[{K},{N}]", "gflop": round(fl / 1e9, 1), "forward": tf_entry(t.ms(fwd, reps), fl),
                       "dgrad": tf_entry(t.ms(dgrad, reps), fl), "wgrad": tf_entry(t.ms(wgrad, reps), fl)}
        if name == "gate_up":
            act.free()
    # vocabulary projection fused with cross-entropy: loss without stored logits; gradient of the logits by a second run
    # of the projection, or in place from stored logits
    tg = ctx.array(np.random.default_rng(0).integers(0, V, M).astype(np.uint32), "u32")
    loss, lse = ctx.empty((1,), "f32"), ctx.empty((M,), "f32")
    flv = 2.0 * M * V * H
    ce_fwd = lambda: ctx._check(lib.b200_vocab_ce_forward(h, big_a.ptr, w.ptr, tg.ptr, loss.ptr, lse.ptr, None, M, V, H, BF))
    ce_fwd_store = lambda: ctx._check(lib.b200_vocab_ce_forward(h, big_a.ptr, w.ptr, tg.ptr, loss.ptr, lse.ptr, big_c.ptr, M, V, H, BF))
    ce_dl = lambda: ctx._check(lib.b200_vocab_ce_backward(h, big_a.ptr, w.ptr, tg.ptr, lse.ptr, big_c.ptr, 0, None, None, M, V, H, BF))
    ce_dl_inplace = lambda: ctx._check(lib.b200_vocab_ce_backward(h, big_a.ptr, w.ptr, tg.ptr, lse.ptr, big_c.ptr, 1, None, None, M, V, H, BF))
    _fill(ctx, bridge, big_a, 3, 0.05)      # keeps the logits of the timed runs in a sane range
    gemms["vocab_ce_fused"] = {"loss_forward_no_logits": tf_entry(t.ms(ce_fwd, reps), flv), "loss_forward_storing_logits": tf_entry(t.ms(ce_fwd_store, reps), flv),
                               "dlogits_by_second_projection": tf_entry(t.ms(ce_dl, reps), flv)}
    gb = lambda ms, nbytes: {"ms": round(ms, 4), "gbs": round(nbytes / (ms / 1e3) / 1e9, 1), "frac_of_hbm": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm"], 3),
                             "mbytes": round(nbytes / 1e6, 1)}
    bw = {}
    bw["vocab_ce_dlogits_in_place"] = gb(t.ms(ce_dl_inplace, reps), 2.0 * M * V * 2)
    bw["cross_entropy_unfused_in_place"] = gb(t.ms(lambda: ctx._check(lib.b200_cross_entropy(h, big_c.ptr, tg.ptr, loss.ptr, big_c.ptr, M, V, BF)), reps), 3.0 * M * V * 2)
    xs = M * H * 2          # one [M, H] bf16 array
    a_, b_, c_, d_ = big_a.ptr, big_a.at(M * H), big_c.ptr, big_c.at(M * H)
    e_ = big_c.at(2 * M * H)
    wn = w.ptr
    bw["rms_norm_forward"] = gb(t.ms(lambda: ctx._check(lib.b200_rms_norm_forward(h, a_, c_, wn, None, 1e-5, M, H, BF)), reps), 2 * xs)
    bw["fused_add_norm"] = gb(t.ms(lambda: ctx._check(lib.b200_fused_add_norm(h, a_, b_, wn, c_, M, H, 1e-5, BF)), reps), 4 * xs)
    bw["rms_norm_backward"] = gb(t.ms(lambda: ctx._check(lib.b200_rms_norm_backward(h, a_, b_, wn, c_, None, 1e-5, M, H, BF)), reps), 3 * xs)
    bw["fused_backward_add_norm"] = gb(t.ms(lambda: ctx._check(lib.b200_fused_backward_add_norm(h, a_, b_, wn, d_, c_, M, H, 1e-5, BF)), reps), 4 * xs)
    n_act = M * I
    bw["swiglu_forward"] = gb(t.ms(lambda: ctx._check(lib.b200_swiglu_forward(h, big_a.ptr, big_a.at(n_act), big_c.ptr, n_act, BF)), reps), 3 * n_act * 2)
    bw["swiglu_backward"] = gb(t.ms(lambda: ctx._check(lib.b200_swiglu_backward(h, big_a.ptr, big_a.at(n_act), big_a.at(2 * n_act), big_c.ptr, big_c.at(n_act), n_act, BF)), reps), 5 * n_act * 2)
    cos, sin = ctx.rope_tables(MODEL["S"], MODEL["hd"])
    nq, nk = MICRO_BATCH * MODEL["nH"] * MODEL["S"] * MODEL["hd"], MICRO_BATCH * MODEL["nKV"] * MODEL["S"] * MODEL["hd"]
    bw["rope_forward_q_and_k"] = gb(t.ms(lambda: ctx._check(lib.b200_rope_forward(h, big_a.ptr, big_a.at(nq), cos.ptr, sin.ptr, MICRO_BATCH, MODEL["nH"], MODEL["nKV"], MODEL["S"], MODEL["hd"], BF)), reps), 2 * (nq + nk) * 2)
    n_adam = 128 * 1024 * 1024
    p32 = _fill(ctx, bridge, ctx.empty((n_adam,), "f32"), 5, 0.02)
    g32 = _fill(ctx, bridge, ctx.empty((n_adam,), "f32"), 6, 0.001)
    m32, v32 = ctx.empty((n_adam,), "f32").zero(), ctx.empty((n_adam,), "f32").zero()
    prm = bridge.AdamWParams(3e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05)
    import ctypes
    bw["adamw_step_fp32_master_bf16_shadow"] = gb(t.ms(lambda: ctx._check(lib.b200_adamw_step(h, p32.ptr, g32.ptr, m32.ptr, v32.ptr, big_c.ptr, n_adam, ctypes.byref(prm))), reps), 30.0 * n_adam)
    launches = ctx.launch_count() - l0
    for a in (big_a, big_c, w, c32, tg, loss, lse, cos, sin, p32, g32, m32, v32):
        a.free()
    return {"workload": f"per-op figures at M = {M} tokens, d_model {H}, ffn {I}, vocab {V}, bf16 (fp32 weight gradients)",
            "gemm_tflops": gemms, "bandwidth_gbs": bw, "launches_timed_per_op": reps, "gpu_launches": int(launches),
            "peaks": pk, "bytes_rule": "each input read once + each output written once; cross_entropy_unfused = 3 x logits (2 reads + 1 write)"}


def run_ops(args):
    import torch
    bridge = importlib.import_module(PKG + ".bridge")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    ctx = bridge.Context(local)
    att = attention_metrics(ctx, bridge, torch, cpu_check=not args.no_cpu_baseline)
    ops = ops_metrics(ctx, bridge, torch)
    ctx.close()
    print(json.dumps({"metric": "attention_fwd_bwd_tflops", "value": att["forward_backward"]["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
                      "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "config": {"workload": att["workload"]},
                      "attention": att, "ops": ops}))


def run_trace(args):
    """In-step device time per launch site: an event after every kernel launch of the library during `--steps` training
    steps (after `--warmup` untraced ones); the time between consecutive events goes to the later launch's source line, or
    to the GEMM's shape.  Prints the table (development aid; the events themselves cost about 1 % of the step)."""
    import tempfile
    bridge = importlib.import_module(PKG + ".bridge")
    synth = importlib.import_module(PKG + ".synth")
    B, S = args.batch, args.seq
    cfg = bridge.Shape(B=B, S=S, H=MODEL["H"], I=MODEL["I"], nH=MODEL["nH"], nKV=MODEL["nKV"], hd=MODEL["hd"], V=MODEL["V"], L=args.layers)
    ctx = bridge.Context(int(os.environ.get("LOCAL_RANK", "0")))
    ctx.lib.b200_internal_trace.argtypes = [bridge._vp, bridge._i]
    ctx.lib.b200_internal_trace_dump.argtypes = [bridge._vp, bridge.C.c_char_p]
    model = bridge.Model(ctx, cfg, "bf16", max_batch=B)
    model.init_synthetic(1234, 0.02)
    tok = synth.token_ids(1000, "tokens", (B, S + 1), MODEL["V"])
    d_tok, d_tgt = ctx.array(np.ascontiguousarray(tok[:, :-1]), "i32"), ctx.array(np.ascontiguousarray(tok[:, 1:]), "i32")
    for _ in range(max(1, args.warmup)):
        model.train_step(d_tok, d_tgt, B, S, **HYPER)
    ctx.sync()
    ctx.lib.b200_internal_trace(ctx.h, 1)
    for _ in range(args.steps):
        model.train_step(d_tok, d_tgt, B, S, **HYPER)
    ctx.lib.b200_internal_trace(ctx.h, 0)
    with tempfile.NamedTemporaryFile("r", suffix=".txt") as f:
        ctx._check(ctx.lib.b200_internal_trace_dump(ctx.h, f.name.encode()))
        print(f"# {args.steps} traced steps, {args.layers} layers, batch {B} x seq {S}")
        print(open(f.name).read())
    model.close(); ctx.close()


def dp_check(ctx, bridge, synth, dist, rank, world, local):
    """Data-parallel correctness on the running ranks, at the model's widths with 2 layers and seq 512: every rank takes
    one sequence, gradients are averaged by the engine's NCCL exchange; rank 0 also runs the engine without NCCL on the
    concatenated batch.  The averaged loss and the exchanged gradients must equal the single-device ones."""
    S = 512
    m = dict(MODEL)
    one = bridge.Shape(B=1, S=S, H=m["H"], I=m["I"], nH=m["nH"], nKV=m["nKV"], hd=m["hd"], V=m["V"], L=2)
    tok = synth.token_ids(77, "dp_tokens", (world, S + 1), m["V"])
    mine = tok[rank:rank + 1]
    model = bridge.Model(ctx, one, "bf16", max_batch=1)
    model.init_synthetic(4321, 0.02)
    ids = [bridge.dp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    model.dp_init(ids[0], rank, world)
    loss = model.loss_and_grads_host(np.ascontiguousarray(mine[:, :-1]), np.ascontiguousarray(mine[:, 1:]))
    grads = model.read_grads() if rank == 0 else None
    model.close()
    losses = [None] * world
    dist.all_gather_object(losses, float(loss))
    out = None
    if rank == 0:
        full = bridge.Shape(B=world, S=S, H=m["H"], I=m["I"], nH=m["nH"], nKV=m["nKV"], hd=m["hd"], V=m["V"], L=2)
        single = bridge.Model(ctx, full, "bf16", max_batch=world)
        single.init_synthetic(4321, 0.02)
        loss_all = single.loss_and_grads_host(np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:]))
        g_all = single.read_grads()
        single.close()
        num = float(np.linalg.norm(grads.astype(np.float64) - g_all)); den = float(np.linalg.norm(g_all.astype(np.float64)))
        out = {"loss_mean_over_ranks": float(np.mean(losses)), "loss_single_device_whole_batch": float(loss_all),
               "loss_rel_diff": abs(float(np.mean(losses)) - loss_all) / abs(loss_all), "grad_rel_diff": num / den,
               "config": f"2 layers at the model's widths, seq {S}, one sequence per rank; gradients after the NCCL exchange vs a "
                         "single-device run on the concatenated batch (bf16: tolerance 2e-2)"}
    return out


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
    dpc = dp_check(ctx, bridge, synth, dist, rank, world, local) if world > 1 else None
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
    # The same K steps once more, now with a CUDA event pair around every tensor-core GEMM launch (the roofline's kernel
    # time).  The events sit between kernels and keep a kernel's set-up from overlapping its predecessor's tail, so the
    # headline region above runs without them; the clock sampler covers both regions.
    ctx.profile_gemm(True)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record(stream)
    for _ in range(args.steps):
        step_dev()
    p1.record(stream)
    barrier()
    ms_profiled = p0.elapsed_time(p1)
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
        # every replica has applied the same averaged gradients to the same weights: fixed-order checksums of the fp32
        # masters must be bit-identical on all ranks
        sums = [None] * world
        dist.all_gather_object(sums, (model.param_checksum(), float(loss_host)))
        if rank == 0:
            ref = sums[0][0]
            dpc = dict(dpc or {})
            dpc["replicas_identical"] = all(c[0] == ref for c in sums)
            dpc["max_rel_diff"] = max(abs(c[0][1] - ref[1]) / abs(ref[1]) for c in sums)
            dpc["weights_sum_sq_rank0"] = ref[1]
            dpc["last_loss_per_rank"] = [c[1] for c in sums]
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
            "config": make_config(world, B, S, args.layers),
            "mfu": {"algorithmic_tflops_per_gpu": fpt * B * S * args.steps / (ms / 1000.0) / 1e12,
                    "six_n_tflops_per_gpu": 6.0 * n_params(mcfg) * B * S * args.steps / (ms / 1000.0) / 1e12,
                    "frac_of_measured_sustained_bf16": fpt * B * S * args.steps / (ms / 1000.0) / 1e12 / peak,
                    "frac_of_nominal_2250": fpt * B * S * args.steps / (ms / 1000.0) / 1e12 / 2250.0},
            "roofline": {"kernel": "gemm_tc2_kernel / gemm_tc_kernel (tcgen05 bf16 GEMM: all projection and vocab GEMMs, fwd + dgrad + wgrad)",
                         "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (achieved / peak) if achieved else None, "peak_source": peak_src,
                         "launches_timed": gemm_n, "share_of_step_time": gemm_ms / ms_profiled if ms_profiled > 0 else None,
                         "timed_in": f"a second pass of the same {args.steps} steps with an event pair around every GEMM launch "
                                     f"({ms_profiled / args.steps:.2f} ms per step with the events, {ms / args.steps:.2f} without)",
                         "traffic": GEMM_DRAM_BYTES_PER_LAUNCH, "traffic_source": GEMM_TRAFFIC_SOURCE,
                         "algorithmic_bytes_per_launch": GEMM_ALGO_BYTES_PER_LAUNCH},
            "e2e": {"value": tokens_total / e2e_s, "unit": UNIT, "h2d_bytes_per_step": int(2 * B * S * 4),
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches), "clocks": clocks, "loss": {"device_path": loss_dev, "host_path": loss_host},
        }
        if dpc is not None:
            out["dp_check"] = dpc
        if not args.no_cpu_baseline and world == 1:
            out["cpu_baseline"] = cpu_baseline()
    model.close()
    if rank == 0 and world == 1 and not args.no_ops:
        out["attention"] = attention_metrics(ctx, bridge, torch, cpu_check=not args.no_cpu_baseline)
        out["ops"] = ops_metrics(ctx, bridge, torch)
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
    ap.add_argument("--no-ops", action="store_true", help="skip the attention / per-op figures appended to the 1-GPU line")
    ap.add_argument("--workload", default="train", choices=["train", "decode", "ops", "trace"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.workload == "ops":
        run_ops(args)
    elif args.workload == "trace":
        run_trace(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
