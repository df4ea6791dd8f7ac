"""Pins the CPU checker (oracle/block_oracle.c) before anything is trusted to it:
  1. the scalar golden values held by the reference's own unit tests,
  2. the committed fixtures produced by the reference's own C++ CPU ops
     (tests/golden/make_golden.py), and
  3. when oracle/_ref has been built on this machine, the reference library
     itself on fresh seeded inputs.
"""
import importlib
import math
import os

import numpy as np
import pytest

from oracle import oracle

synth = importlib.import_module("large-language-model_b200.synth")
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu_ops.npz"))
SEED = 20240
TOY = dict(B=2, S=8, H=32, I=48, nH=4, nKV=2, hd=8, V=64, L=2)
C1 = dict(B=2, S=128, H=256, I=688, nH=8, nKV=2, hd=32, V=4096, L=1)


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30))


def digest(a, n=256):
    a = np.asarray(a, np.float32).ravel()
    idx = np.linspace(0, a.size - 1, n).astype(np.int64)
    return np.concatenate([[np.sqrt(np.sum(a.astype(np.float64) ** 2)), a.astype(np.float64).sum()],
                           a[idx].astype(np.float64)])


def close_digest(a, gold, tol=2e-5):
    d = digest(a)
    assert abs(d[0] - gold[0]) <= tol * abs(gold[0]) + 1e-12, (d[0], gold[0])
    assert rel(d[2:], gold[2:]) <= tol * 5, rel(d[2:], gold[2:])


def inputs(cfg):
    params = synth.model_params(SEED, cfg)
    tokens = synth.token_ids(SEED, "tokens", (cfg.B, cfg.S + 1), cfg.V)
    return params, np.ascontiguousarray(tokens[:, :-1]), np.ascontiguousarray(tokens[:, 1:])


# ---- 1. known answers from the reference's unit tests -------------------
def test_rmsnorm_known_answers(orc):
    # cpp/tests/test_rmsnorm.cpp:49,75-78 and weight scaling :110-129
    x = np.array([[0.3, 0.9], [-0.7, 0.4]], np.float32)
    y = orc.rms_norm_forward(x, np.ones(2, np.float32))
    np.testing.assert_allclose(y.ravel(), [0.447208, 1.341625, -1.22786, 0.701635], atol=2e-5)
    y2 = orc.rms_norm_forward(x, np.array([2.0, 0.5], np.float32))
    np.testing.assert_allclose(y2[0], [0.447208 * 2, 1.341625 * 0.5], atol=4e-5)


def test_rope_known_answers(orc):
    # cpp/tests/test_rope.cpp:68-97 tables; :115-136 rotation x0*c - x1*s at pos 1
    c, s = orc.rope_tables(4, 8)
    assert c.shape == (4, 4)
    np.testing.assert_allclose(c[0], 1.0)
    np.testing.assert_allclose(s[0], 0.0)
    assert abs(c[1, 0] - math.cos(1.0)) < 1e-6 and abs(s[1, 0] - math.sin(1.0)) < 1e-6
    q = np.tile(np.arange(1, 9, dtype=np.float32), (1, 1, 2, 1))
    r = orc.rope(q, c, s)
    np.testing.assert_allclose(r[0, 0, 0], np.arange(1, 9), atol=1e-6)      # pos 0 is the identity
    assert abs(r[0, 0, 1, 0] - (1.0 * math.cos(1.0) - 2.0 * math.sin(1.0))) < 1e-5
    back = orc.rope(r, c, s, backward=True)
    np.testing.assert_allclose(back, q, atol=1e-5)


def test_swiglu_known_answers(orc):
    # cpp/tests/test_activations.cpp:48-75: silu(2)=1.76159, swiglu([0,2],[10,5])=[0,8.80797]
    y = orc.swiglu_forward(np.array([0.0, 2.0], np.float32), np.array([10.0, 5.0], np.float32))
    np.testing.assert_allclose(y, [0.0, 8.80797], atol=1e-5)
    y1 = orc.swiglu_forward(np.array([0.0, 2.0], np.float32), np.ones(2, np.float32))
    assert abs(y1[1] - 1.76159) < 1e-5


def test_loss_known_answers(orc):
    # cpp/tests/test_loss.cpp:56-101: uniform logits -> ln 4, grad [1/4,1/4,-3/4,1/4]; 1000-valued logits finite
    loss, d = orc.cross_entropy(np.zeros((1, 4), np.float32), [2])
    assert abs(loss - math.log(4.0)) < 1e-5
    np.testing.assert_allclose(d[0], [0.25, 0.25, -0.75, 0.25], atol=1e-6)
    loss, _ = orc.cross_entropy(np.full((1, 4), 1000.0, np.float32), [1])
    assert math.isfinite(loss) and abs(loss - math.log(4.0)) < 1e-5


def test_matmul_known_answers(orc):
    # cpp/tests/test_math_ops.cpp:167-188
    m = orc.gemm(np.arange(1, 7, dtype=np.float32).reshape(2, 3), np.arange(7, 13, dtype=np.float32).reshape(3, 2), 2, 2, 3)
    np.testing.assert_array_equal(m, [[58, 64], [139, 154]])


def test_attention_properties(orc):
    # property checks of cpp/tests/test_attention.cpp: causal-mask leak (:99-115),
    # identical tokens -> identical outputs (:321-334), zero upstream grad -> zero grads,
    # 2x upstream grad -> 2x dx (:513-535)
    cfg = oracle.Config(B=1, S=6, H=16, I=32, nH=4, nKV=2, hd=4)
    W = [synth.normal(7, n, s, 0.3) for n, s in (("q", (16, 16)), ("k", (16, 8)), ("v", (16, 8)), ("o", (16, 16)))]
    x = synth.normal(7, "x", (1, 6, 16))
    base = orc.attention_layer(cfg, x, *W)
    x2 = x.copy()
    x2[0, 4:] += 5.0                                  # change the future only
    np.testing.assert_allclose(orc.attention_layer(cfg, x2, *W)[0, :4], base[0, :4], atol=1e-6)
    g = synth.normal(7, "g", (1, 6, 16))
    _, gx, gW = orc.attention_layer(cfg, x, *W, gout=g)
    _, gx2, gW2 = orc.attention_layer(cfg, x, *W, gout=2 * g)
    np.testing.assert_allclose(gx2, 2 * gx, rtol=1e-5, atol=1e-7)
    _, gx0, gW0 = orc.attention_layer(cfg, x, *W, gout=np.zeros_like(g))
    assert not gx0.any() and not any(a.any() for a in gW0)
    assert all(np.abs(a).max() > 0 for a in gW)


def test_layer_gradients_against_finite_differences(orc):
    # the integration check of cpp/tests/test_backward.cpp:105-151, tightened
    cfg = oracle.Config(B=2, S=5, H=16, I=24, nH=4, nKV=2, hd=4, V=11, L=2)
    params = synth.model_params(3, cfg, std=0.3).astype(np.float32)
    tok = synth.token_ids(3, "t", (2, 6), 11)
    t, y = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
    _, grads, _ = orc.model_loss_and_grads(cfg, t, y, params)
    rng = np.random.default_rng(0)
    for i in rng.choice(params.size, 24, replace=False):
        p = params.copy(); p[i] += 2e-3
        lp, _, _ = orc.model_loss_and_grads(cfg, t, y, p, want_grads=False)
        p[i] -= 4e-3
        lm, _, _ = orc.model_loss_and_grads(cfg, t, y, p, want_grads=False)
        num = (lp - lm) / 4e-3
        assert abs(num - grads[i]) < 2e-3 + 2e-2 * abs(num), (i, num, grads[i])


# ---- 2. committed fixtures from the reference's own CPU ops --------------
def test_primitives_match_reference_fixtures(orc):
    x = synth.normal(SEED, "prim.x", (6, 32))
    w = 1.0 + 0.1 * synth.normal(SEED, "prim.w", (32,))
    g = synth.normal(SEED, "prim.g", (6, 32))
    assert rel(orc.rms_norm_forward(x, w), GOLD["rms_fwd"]) < 1e-6
    dx, dw = orc.rms_norm_backward(g, x, w)
    assert rel(dx, GOLD["rms_bwd_dx"]) < 1e-6 and rel(dw, GOLD["rms_bwd_dw"]) < 1e-6
    c, s = orc.rope_tables(16, 8)
    assert np.array_equal(c, GOLD["rope_cos"]) and np.array_equal(s, GOLD["rope_sin"])
    t4 = synth.normal(SEED, "prim.t4", (2, 3, 16, 8))
    assert np.array_equal(orc.rope(t4, c, s), GOLD["rope_fwd"])
    assert np.array_equal(orc.rope(t4, c, s, backward=True), GOLD["rope_bwd"])
    gate, up, dy = (synth.normal(SEED, "prim." + n, (200,)) for n in ("gate", "up", "dy"))
    assert rel(orc.swiglu_forward(gate, up), GOLD["swiglu_fwd"]) < 1e-6
    dg, du = orc.swiglu_backward(dy, gate, up)
    assert rel(dg, GOLD["swiglu_bwd_dg"]) < 1e-6 and rel(du, GOLD["swiglu_bwd_du"]) < 1e-6
    lg = synth.normal(SEED, "prim.logits", (10, 50), 3.0)
    tg = synth.token_ids(SEED, "prim.tg", (10,), 50)
    loss, dl = orc.cross_entropy(lg, tg)
    assert abs(loss - float(GOLD["ce_loss"])) < 1e-6 and rel(dl, GOLD["ce_dlogits"]) < 1e-6
    A, B_ = synth.normal(SEED, "prim.A", (7, 9)), synth.normal(SEED, "prim.B", (9, 5))
    assert rel(orc.gemm(A, B_, 7, 5, 9), GOLD["gemm_nn"]) < 1e-6
    assert rel(orc.gemm(A, synth.normal(SEED, "prim.Bt", (5, 9)), 7, 5, 9, transB=True), GOLD["gemm_nt"]) < 1e-6
    assert rel(orc.gemm(synth.normal(SEED, "prim.At", (9, 7)), B_, 7, 5, 9, transA=True), GOLD["gemm_tn"]) < 1e-6
    p, gr = synth.normal(SEED, "prim.p", (300,), 0.02), synth.normal(SEED, "prim.gr", (300,), 0.01)
    m0, v0 = 0.001 * synth.normal(SEED, "prim.m", (300,)), np.abs(1e-5 * synth.normal(SEED, "prim.v", (300,)))
    pn, mn, vn = orc.adamw_step(p, gr, m0, v0, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3)
    assert rel(pn, GOLD["adamw_p"]) < 1e-6 and rel(mn, GOLD["adamw_m"]) < 1e-6 and rel(vn, GOLD["adamw_v"]) < 1e-6


def test_toy_compositions_match_reference_fixtures(orc):
    cfg = oracle.Config(**TOY)
    params, tok, tgt = inputs(cfg)
    lp = params[cfg.V * cfg.H: cfg.V * cfg.H + cfg.layer_params]
    W = {k: lp[o:o + int(np.prod(s))].reshape(s) for k, (o, s) in cfg.layer_slices().items()}
    xa = synth.normal(SEED, "toy.x", (cfg.B, cfg.S, cfg.H))
    ga = synth.normal(SEED, "toy.gout", (cfg.B, cfg.S, cfg.H))
    o, gx, gW = orc.attention_layer(cfg, xa, W["Wq"], W["Wk"], W["Wv"], W["Wo"], ga)
    assert rel(o, GOLD["toy_attn_out"]) < 2e-6 and rel(gx, GOLD["toy_attn_gx"]) < 2e-6
    for n, a in zip(("gWq", "gWk", "gWv", "gWo"), gW):
        assert rel(a, GOLD["toy_attn_" + n]) < 2e-6, n
    assert rel(orc.layer_forward(cfg, xa, lp), GOLD["toy_layer_out"]) < 2e-6
    gh, gl = orc.layer_backward(cfg, ga, xa, lp)
    assert rel(gh, GOLD["toy_layer_gh"]) < 2e-6
    gold = GOLD["toy_layer_grads"]
    for k, (off, shp) in cfg.layer_slices().items():
        if k.endswith("norm_w"):
            continue            # the reference computes and then discards norm-weight gradients
        n = int(np.prod(shp))
        assert rel(gl[off:off + n], gold[off:off + n]) < 2e-6, k
    loss, grads, logits = orc.model_loss_and_grads(cfg, tok, tgt, params, want_logits=True)
    assert abs(loss - float(GOLD["toy_model_loss"])) < 2e-6
    assert rel(logits, GOLD["toy_model_logits"]) < 2e-6
    mask = np.ones(cfg.model_params, bool)
    for l in range(cfg.L):
        base = cfg.V * cfg.H + l * cfg.layer_params
        for k, (off, shp) in cfg.layer_slices().items():
            if k.endswith("norm_w"):
                mask[base + off: base + off + cfg.H] = False
    mask[cfg.V * cfg.H + cfg.L * cfg.layer_params: cfg.V * cfg.H + cfg.L * cfg.layer_params + cfg.H] = False
    assert rel(grads[mask], GOLD["toy_model_grads"][mask]) < 2e-6


def test_single_layer_benchmark_config_matches_reference_fixtures(orc):
    cfg = oracle.Config(**C1)
    params, tok, tgt = inputs(cfg)
    lp = params[cfg.V * cfg.H: cfg.V * cfg.H + cfg.layer_params]
    xa = synth.normal(SEED, "c1.x", (cfg.B, cfg.S, cfg.H))
    ga = synth.normal(SEED, "c1.gout", (cfg.B, cfg.S, cfg.H))
    close_digest(orc.layer_forward(cfg, xa, lp), GOLD["c1_layer_out"])
    gh, gl = orc.layer_backward(cfg, ga, xa, lp)
    close_digest(gh, GOLD["c1_layer_gh"])
    for k, (off, shp) in cfg.layer_slices().items():
        if not k.endswith("norm_w"):
            close_digest(gl[off:off + int(np.prod(shp))], GOLD["c1_layer_g_" + k])
    loss, grads, logits = orc.model_loss_and_grads(cfg, tok, tgt, params, want_logits=True)
    assert abs(loss - float(GOLD["c1_model_loss"])) < 1e-5
    close_digest(logits, GOLD["c1_model_logits"])
    close_digest(grads[:cfg.V * cfg.H], GOLD["c1_model_g_emb"])
    close_digest(grads[-cfg.H * cfg.V:], GOLD["c1_model_g_out"])


# ---- 3. the reference library itself, where it has been built -----------
@pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built on this machine")
def test_against_live_reference_library(orc):
    ref = oracle.load_ref()
    cfg = oracle.Config(B=2, S=12, H=48, I=80, nH=6, nKV=3, hd=8, V=96, L=2)
    params = synth.model_params(99, cfg, std=0.1)
    tok = synth.token_ids(99, "t", (2, 13), 96)
    t, y = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
    lo, go, lgo = orc.model_loss_and_grads(cfg, t, y, params, want_logits=True)
    lr, gr, lgr = ref.model_loss_and_grads(cfg, t, y, params, want_logits=True)
    assert abs(lo - lr) < 1e-5 and rel(lgo, lgr) < 2e-6
    nz = gr != 0
    assert rel(go[nz], gr[nz]) < 5e-6
