"""Generates the golden fixtures in this directory from the REFERENCE's own
C++ CPU ops (oracle/_ref/libref_oracle.so, built by oracle/build_ref.sh from
the reference checkout, alias-fixed variant).  Run from the repository root:

    sh oracle/build_ref.sh && python tests/golden/make_golden.py
    (python tests/golden/make_golden.py trainer   regenerates only the checkpoint / schedule fixtures)

The fixtures are what pins oracle/block_oracle.c (tests/test_oracle.py) and,
through it, the CUDA kernels, on machines where the reference checkout is
absent.  Inputs are regenerated from seeds by the test, so only outputs are
stored: full arrays for the toy configuration, and for the single-layer
benchmark configuration (B2 S128 d256 8q/2kv hd32 I688 V4096) a digest per
tensor (L2 norm, sum, 256 evenly strided samples).
"""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402

synth = importlib.import_module("large-language-model_b200.synth")
HERE = os.path.dirname(os.path.abspath(__file__))

TOY = dict(B=2, S=8, H=32, I=48, nH=4, nKV=2, hd=8, V=64, L=2)
C1 = dict(B=2, S=128, H=256, I=688, nH=8, nKV=2, hd=32, V=4096, L=1)
SEED = 20240


def digest(a, n=256):
    a = np.asarray(a, np.float32).ravel()
    idx = np.linspace(0, a.size - 1, n).astype(np.int64)
    return np.concatenate([[np.sqrt(np.sum(a.astype(np.float64) ** 2)), a.astype(np.float64).sum()],
                           a[idx].astype(np.float64)]).astype(np.float64)


def inputs(cfg, seed=SEED):
    params = synth.model_params(seed, cfg)
    tokens = synth.token_ids(seed, "tokens", (cfg.B, cfg.S + 1), cfg.V)
    return params, np.ascontiguousarray(tokens[:, :-1]), np.ascontiguousarray(tokens[:, 1:])


def main():
    ref = oracle.load_ref()
    out = {}
    # --- primitive ops on small seeded inputs (full arrays) -------------
    x = synth.normal(SEED, "prim.x", (6, 32))
    w = 1.0 + 0.1 * synth.normal(SEED, "prim.w", (32,))
    g = synth.normal(SEED, "prim.g", (6, 32))
    out["rms_fwd"] = ref.rms_norm_forward(x, w)
    dx, dw = ref.rms_norm_backward(g, x, w)
    out["rms_bwd_dx"], out["rms_bwd_dw"] = dx, dw
    c, s = ref.rope_tables(16, 8)
    out["rope_cos"], out["rope_sin"] = c, s
    t4 = synth.normal(SEED, "prim.t4", (2, 3, 16, 8))
    out["rope_fwd"] = ref.rope(t4, c, s)
    out["rope_bwd"] = ref.rope(t4, c, s, backward=True)
    gate, up, dy = (synth.normal(SEED, "prim." + n, (200,)) for n in ("gate", "up", "dy"))
    out["swiglu_fwd"] = ref.swiglu_forward(gate, up)
    out["swiglu_bwd_dg"], out["swiglu_bwd_du"] = ref.swiglu_backward(dy, gate, up)
    lg = synth.normal(SEED, "prim.logits", (10, 50), 3.0)
    tg = synth.token_ids(SEED, "prim.tg", (10,), 50)
    loss, dl = ref.cross_entropy(lg, tg)
    out["ce_loss"], out["ce_dlogits"] = np.float32(loss), dl
    A, B_ = synth.normal(SEED, "prim.A", (7, 9)), synth.normal(SEED, "prim.B", (9, 5))
    out["gemm_nn"] = ref.gemm(A, B_, 7, 5, 9)
    out["gemm_nt"] = ref.gemm(A, synth.normal(SEED, "prim.Bt", (5, 9)), 7, 5, 9, transB=True)
    out["gemm_tn"] = ref.gemm(synth.normal(SEED, "prim.At", (9, 7)), B_, 7, 5, 9, transA=True)
    p, gr = synth.normal(SEED, "prim.p", (300,), 0.02), synth.normal(SEED, "prim.gr", (300,), 0.01)
    m0, v0 = 0.001 * synth.normal(SEED, "prim.m", (300,)), np.abs(1e-5 * synth.normal(SEED, "prim.v", (300,)))
    out["adamw_p"], out["adamw_m"], out["adamw_v"] = ref.adamw_step(p, gr, m0, v0, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3)
    # --- attention sub-layer, decoder layer, whole model: toy config ----
    cfg = oracle.Config(**TOY)
    params, tok, tgt = inputs(cfg)
    sl = cfg.layer_slices()
    lp = params[cfg.V * cfg.H: cfg.V * cfg.H + cfg.layer_params]
    W = {k: lp[o:o + int(np.prod(s))].reshape(s) for k, (o, s) in sl.items()}
    xa = synth.normal(SEED, "toy.x", (cfg.B, cfg.S, cfg.H))
    ga = synth.normal(SEED, "toy.gout", (cfg.B, cfg.S, cfg.H))
    o, gx, gW = ref.attention_layer(cfg, xa, W["Wq"], W["Wk"], W["Wv"], W["Wo"], ga)
    out["toy_attn_out"], out["toy_attn_gx"] = o, gx
    for n, a in zip(("gWq", "gWk", "gWv", "gWo"), gW):
        out["toy_attn_" + n] = a
    out["toy_layer_out"] = ref.layer_forward(cfg, xa, lp)
    gh, gl = ref.layer_backward(cfg, ga, xa, lp)
    out["toy_layer_gh"], out["toy_layer_grads"] = gh, gl
    loss, grads, logits = ref.model_loss_and_grads(cfg, tok, tgt, params, want_logits=True)
    out["toy_model_loss"], out["toy_model_grads"], out["toy_model_logits"] = np.float32(loss), grads, logits
    # --- single-layer benchmark configuration: digests -------------------
    cfg = oracle.Config(**C1)
    params, tok, tgt = inputs(cfg)
    lp = params[cfg.V * cfg.H: cfg.V * cfg.H + cfg.layer_params]
    xa = synth.normal(SEED, "c1.x", (cfg.B, cfg.S, cfg.H))
    ga = synth.normal(SEED, "c1.gout", (cfg.B, cfg.S, cfg.H))
    out["c1_layer_out"] = digest(ref.layer_forward(cfg, xa, lp))
    gh, gl = ref.layer_backward(cfg, ga, xa, lp)
    out["c1_layer_gh"] = digest(gh)
    for k, (o_, s_) in cfg.layer_slices().items():
        out["c1_layer_g_" + k] = digest(gl[o_:o_ + int(np.prod(s_))])
    loss, grads, logits = ref.model_loss_and_grads(cfg, tok, tgt, params, want_logits=True)
    out["c1_model_loss"] = np.float32(loss)
    out["c1_model_logits"] = digest(logits)
    out["c1_model_g_emb"] = digest(grads[:cfg.V * cfg.H])
    out["c1_model_g_layer"] = digest(grads[cfg.V * cfg.H: cfg.V * cfg.H + cfg.layer_params])
    out["c1_model_g_out"] = digest(grads[-cfg.H * cfg.V:])
    np.savez_compressed(os.path.join(HERE, "reference_cpu_ops.npz"), **out)
    print("wrote", len(out), "arrays;", os.path.getsize(os.path.join(HERE, "reference_cpu_ops.npz")), "bytes")


TINY = dict(B=1, S=4, H=8, I=12, nH=2, nKV=1, hd=4, V=11, L=2)
LR_CASES = [(w, mx, lmax, lmin) for (w, mx) in ((10, 100), (0, 7), (2000, 100000), (5, 5)) for (lmax, lmin) in ((3e-4, 3e-5), (1e-3, 0.0))]
LR_STEPS = [0, 1, 2, 4, 5, 6, 7, 9, 10, 11, 50, 99, 100, 101, 1999, 2000, 2001, 51000, 99999, 100000, 123456]


def trainer_files():
    """The reference's Checkpoint::save output for a tiny seeded model (the two files are committed as they are)
    and Trainer::get_scheduled_lr on a grid of steps / configurations."""
    ref = oracle.load_ref()
    cfg = oracle.Config(**TINY)
    params = synth.model_params(SEED, cfg, std=0.5)
    m = synth.normal(SEED, "ckpt.m", (cfg.model_params,), 0.01)
    v = np.abs(synth.normal(SEED, "ckpt.v", (cfg.model_params,), 1e-4))
    ref.checkpoint_save(cfg, os.path.join(HERE, "ckpt_tiny.safetensors"), params, m, v, 1234)
    lr = np.array([[ref.scheduled_lr(st, *case) for st in LR_STEPS] for case in LR_CASES], np.float32)
    np.savez_compressed(os.path.join(HERE, "reference_trainer.npz"), lr=lr)
    print("wrote ckpt_tiny.safetensors (+ .opt) and", lr.size, "schedule values")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "trainer":
        trainer_files()
    else:
        main()
        trainer_files()
