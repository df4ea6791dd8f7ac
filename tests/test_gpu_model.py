"""Decoder layer and whole-model parity of the device-resident engine against the CPU checker
and the committed reference fixtures: the single-layer benchmark configuration in fp32
(rel-err <= 1e-4 on every output and gradient), bf16 (<= 2e-2), AdamW steps, and training."""
import os

import numpy as np
import pytest

from gpu_util import BF16_TOL, FP32_TOL, bridge, ctx, rel, synth  # noqa: F401
from oracle import oracle

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu_ops.npz"))
SEED = 20240
TOY = dict(B=2, S=8, H=32, I=48, nH=4, nKV=2, hd=8, V=64, L=2)
C1 = dict(B=2, S=128, H=256, I=688, nH=8, nKV=2, hd=32, V=4096, L=1)


def inputs(cfg, seed=SEED):
    params = synth.model_params(seed, cfg)
    tokens = synth.token_ids(seed, "tokens", (cfg.B, cfg.S + 1), cfg.V)
    return params, np.ascontiguousarray(tokens[:, :-1]), np.ascontiguousarray(tokens[:, 1:])


def trainable_mask(cfg):
    mask = np.ones(cfg.model_params, bool)
    for l in range(cfg.L):
        base = cfg.V * cfg.H + l * cfg.layer_params
        for k, (off, shp) in cfg.layer_slices().items():
            if k.endswith("norm_w"):
                mask[base + off: base + off + cfg.H] = False
    e = cfg.V * cfg.H + cfg.L * cfg.layer_params
    mask[e:e + cfg.H] = False
    return mask


def digest(a, n=256):
    a = np.asarray(a, np.float32).ravel()
    idx = np.linspace(0, a.size - 1, n).astype(np.int64)
    return np.concatenate([[np.sqrt(np.sum(a.astype(np.float64) ** 2)), a.astype(np.float64).sum()], a[idx].astype(np.float64)])


# d_model 2048 in fp32: the row shape at which the norm kernels split a row over four warps
WIDE = dict(B=1, S=32, H=2048, I=256, nH=16, nKV=4, hd=128, V=128, L=1)


@pytest.mark.parametrize("cfgd", [TOY, C1, WIDE], ids=["toy", "single_layer_benchmark_config", "d_model_2048"])
def test_fp32_model_loss_logits_and_every_gradient(ctx, orc, cfgd):
    cfg = oracle.Config(**cfgd)
    params, tok, tgt = inputs(cfg)
    loss_ref, grads_ref, logits_ref = orc.model_loss_and_grads(cfg, tok, tgt, params, want_logits=True)
    model = bridge.Model(ctx, cfg, "f32")
    model.load_params(params)
    np.testing.assert_array_equal(model.read_params(), params)              # import/export is lossless
    logits = model.forward(ctx.array(tok, "i32"), cfg.B, cfg.S).download()
    assert rel(logits, logits_ref) < FP32_TOL
    loss = model.loss_and_grads_host(tok, tgt)
    assert abs(loss - loss_ref) < 1e-5 * max(1.0, abs(loss_ref))
    grads = model.read_grads()
    mask = trainable_mask(cfg)
    lp, e = cfg.layer_params, cfg.V * cfg.H
    assert rel(grads[:e], grads_ref[:e]) < FP32_TOL                        # embedding
    assert rel(grads[-cfg.H * cfg.V:], grads_ref[-cfg.H * cfg.V:]) < FP32_TOL   # output projection
    for l in range(cfg.L):
        for k, (off, shp) in cfg.layer_slices().items():
            if k.endswith("norm_w"):
                continue
            n = int(np.prod(shp))
            sl = slice(e + l * lp + off, e + l * lp + off + n)
            assert rel(grads[sl], grads_ref[sl]) < FP32_TOL, (l, k)
    assert not grads[~mask].any()           # norm weights are not trained (cpp/src/Trainer.cpp:195-205)
    if cfgd is C1:                          # and against the reference's own CPU ops (committed digests)
        assert abs(loss - float(GOLD["c1_model_loss"])) < 1e-4
        d = digest(grads[:e]); g = GOLD["c1_model_g_emb"]
        assert abs(d[0] - g[0]) < 1e-4 * g[0] and rel(d[2:], g[2:]) < 1e-3
        d = digest(logits); g = GOLD["c1_model_logits"]
        assert abs(d[0] - g[0]) < 1e-4 * g[0] and rel(d[2:], g[2:]) < 1e-4
    model.close()


@pytest.mark.parametrize("cfgd", [TOY, C1], ids=["toy", "single_layer_benchmark_config"])
def test_fp32_single_layer_forward_backward(ctx, orc, cfgd):
    cfg = oracle.Config(**{**cfgd, "L": 1})
    params, _, _ = inputs(cfg)
    lp = params[cfg.V * cfg.H: cfg.V * cfg.H + cfg.layer_params]
    tag = "toy" if cfgd is TOY else "c1"
    x = synth.normal(SEED, tag + ".x", (cfg.B, cfg.S, cfg.H))
    g = synth.normal(SEED, tag + ".gout", (cfg.B, cfg.S, cfg.H))
    model = bridge.Model(ctx, cfg, "f32")
    model.load_params(params)
    out = model.layer_forward(0, ctx.array(x), cfg.B, cfg.S).download()
    assert rel(out, orc.layer_forward(cfg, x, lp)) < FP32_TOL
    gh = model.layer_backward(0, ctx.array(g), cfg.B, cfg.S).download()
    egh, egl = orc.layer_backward(cfg, g, x, lp)
    assert rel(gh, egh) < FP32_TOL
    grads = model.read_grads()[cfg.V * cfg.H: cfg.V * cfg.H + cfg.layer_params]
    for k, (off, shp) in cfg.layer_slices().items():
        if not k.endswith("norm_w"):
            n = int(np.prod(shp))
            assert rel(grads[off:off + n], egl[off:off + n]) < FP32_TOL, k
    if cfgd is C1:
        d, gd = digest(out), GOLD["c1_layer_out"]
        assert abs(d[0] - gd[0]) < 1e-4 * gd[0] and rel(d[2:], gd[2:]) < 1e-4
        d, gd = digest(gh), GOLD["c1_layer_gh"]
        assert abs(d[0] - gd[0]) < 1e-4 * gd[0] and rel(d[2:], gd[2:]) < 1e-4
    model.close()


@pytest.mark.parametrize("cfgd", [dict(B=2, S=128, H=256, I=688, nH=8, nKV=2, hd=32, V=4096, L=2),
                                  dict(B=2, S=256, H=512, I=1024, nH=4, nKV=2, hd=128, V=2048, L=2),
                                  # enough 256x256 tile pairs for the two-CTA GEMM with the SwiGLU epilogues (forward and backward)
                                  dict(B=2, S=1024, H=256, I=1280, nH=2, nKV=1, hd=128, V=1024, L=1),
                                  # the benchmark's d_model (norm rows of 1024 / 2048: one and two warps per row)
                                  dict(B=1, S=128, H=1024, I=512, nH=8, nKV=2, hd=128, V=512, L=2),
                                  dict(B=1, S=128, H=2048, I=512, nH=16, nKV=4, hd=128, V=512, L=2)],
                         ids=["hd32", "hd128", "two_cta_fused_swiglu", "d_model_1024", "d_model_2048"])
def test_bf16_model_against_fp32_checker(ctx, orc, cfgd):
    cfg = oracle.Config(**cfgd)
    params, tok, tgt = inputs(cfg, seed=9)
    params = synth.bf16_round(params)
    loss_ref, grads_ref, logits_ref = orc.model_loss_and_grads(cfg, tok, tgt, params, want_logits=True)
    model = bridge.Model(ctx, cfg, "bf16")
    model.load_params(params)
    logits = model.forward(ctx.array(tok, "i32"), cfg.B, cfg.S).download()
    assert rel(logits, logits_ref) < BF16_TOL
    loss = model.loss_and_grads_host(tok, tgt)
    assert abs(loss - loss_ref) < 2e-3 * abs(loss_ref)
    grads = model.read_grads()
    lp, e = cfg.layer_params, cfg.V * cfg.H
    assert rel(grads[:e], grads_ref[:e]) < BF16_TOL
    assert rel(grads[-cfg.H * cfg.V:], grads_ref[-cfg.H * cfg.V:]) < BF16_TOL
    for l in range(cfg.L):
        for k, (off, shp) in cfg.layer_slices().items():
            if k.endswith("norm_w"):
                continue
            n = int(np.prod(shp))
            sl = slice(e + l * lp + off, e + l * lp + off + n)
            assert rel(grads[sl], grads_ref[sl]) < BF16_TOL, (l, k, rel(grads[sl], grads_ref[sl]))
    # the same step with the single-CTA GEMM forced: no fused SwiGLU epilogues, separate kernels instead
    ctx.lib.b200_internal_set_gemm_2cta.argtypes = [bridge._vp, bridge._i]
    ctx.lib.b200_internal_set_gemm_2cta(ctx.h, 0)
    try:
        loss1 = model.loss_and_grads_host(tok, tgt)
        grads1 = model.read_grads()
    finally:
        ctx.lib.b200_internal_set_gemm_2cta(ctx.h, 1)
    # the two-CTA epilogue activates the fp32 accumulators, the separate kernel the bf16-rounded products: the two
    # routes differ by one bf16 rounding of gate and up, both stay inside the gate against the checker
    assert abs(loss1 - loss) < 2e-4 * abs(loss) and rel(grads1, grads) < 6e-3, (loss1, loss, rel(grads1, grads))
    assert rel(grads1[-cfg.H * cfg.V:], grads_ref[-cfg.H * cfg.V:]) < BF16_TOL and rel(grads1[:e], grads_ref[:e]) < BF16_TOL
    model.close()


def test_bit_reproducible_gradient_mode(ctx, orc):
    """With the reproducible paths on (no split-K, attention backward writes dQ per key tile and adds the tiles in order,
    the embedding gradient is added token by token) two runs give bit-identical gradients; they agree with the
    default paths, whose atomics add the same terms in a varying order, and with the checker."""
    cfg = oracle.Config(B=2, S=512, H=256, I=512, nH=2, nKV=1, hd=128, V=1024, L=2)     # 4 key tiles; wgrads with a 1024-deep K
    params, tok, tgt = inputs(cfg, seed=13)
    tok[:, ::3] = tok[:, :1]                                   # repeated ids: several tokens add into one embedding row
    params = synth.bf16_round(params)
    _, grads_ref, _ = orc.model_loss_and_grads(cfg, tok, tgt, params, want_logits=True)
    model = bridge.Model(ctx, cfg, "bf16")
    model.load_params(params)
    ctx.lib.b200_internal_set_deterministic.argtypes = [bridge._vp, bridge._i]
    try:
        ctx.lib.b200_internal_set_deterministic(ctx.h, 1)
        loss_a = model.loss_and_grads_host(tok, tgt); ga = model.read_grads()
        loss_b = model.loss_and_grads_host(tok, tgt); gb = model.read_grads()
        assert loss_a == loss_b
        np.testing.assert_array_equal(ga, gb)
        ctx.lib.b200_internal_set_deterministic(ctx.h, 0)
        loss_c = model.loss_and_grads_host(tok, tgt); gc = model.read_grads()
        assert loss_c == loss_a and rel(gc, ga) < 1e-5
        nz = grads_ref != 0
        assert rel(ga[nz & (ga != 0)], grads_ref[nz & (ga != 0)]) < BF16_TOL
    finally:
        ctx.lib.b200_internal_set_deterministic(ctx.h, 0)
        model.close()


def test_adamw_training_steps_match_the_checker_and_reduce_the_loss(ctx, orc):
    cfg = oracle.Config(B=2, S=16, H=64, I=96, nH=4, nKV=2, hd=16, V=96, L=2)
    params, tok, tgt = inputs(cfg, seed=3)
    model = bridge.Model(ctx, cfg, "f32")
    model.load_params(params)
    p = params.copy()
    m, v = np.zeros_like(p), np.zeros_like(p)
    mask = trainable_mask(cfg)
    losses = []
    for step in range(1, 4):
        loss = model.train_step_host(tok, tgt, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
        l_ref, g_ref, _ = orc.model_loss_and_grads(cfg, tok, tgt, p)
        assert abs(loss - l_ref) < 1e-4 * max(1, abs(l_ref))
        pn, mn, vn = orc.adamw_step(p, g_ref, m, v, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
        p = np.where(mask, pn, p); m = np.where(mask, mn, m); v = np.where(mask, vn, v)
        losses.append(loss)
    assert rel(model.read_params(), p) < 1e-4
    for _ in range(40):       # overfit check of cpp/tests/test_trainer.cpp:179-252
        loss = model.train_step_host(tok, tgt, lr=1e-2)
    assert loss < 0.5 * losses[0]
    model.close()


def test_global_norm_gradient_clipping_of_the_optimizer_step(ctx, orc):
    """python/apple-silicon/src/pre-training/train.py:858-867: norm over all gradients; scale max/(norm + 1e-6) when it
    exceeds the bound.  The step with clipping equals the checker's AdamW on the scaled gradients; a bound above the
    norm changes nothing."""
    cfg = oracle.Config(B=2, S=16, H=64, I=96, nH=4, nKV=2, hd=16, V=96, L=2)
    params, tok, tgt = inputs(cfg, seed=4)
    mask = trainable_mask(cfg)
    _, g_ref, _ = orc.model_loss_and_grads(cfg, tok, tgt, params)
    norm_ref = float(np.sqrt(np.sum(g_ref[mask].astype(np.float64) ** 2)))
    for bound in (0.25 * norm_ref, 4.0 * norm_ref):
        model = bridge.Model(ctx, cfg, "f32")
        model.load_params(params)
        model.set_grad_clip(bound)
        model.train_step_host(tok, tgt, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
        norm, factor = model.last_grad_norm()
        exp_factor = bound / (norm_ref + 1e-6) if norm_ref > bound else 1.0
        assert abs(norm - norm_ref) < 1e-4 * norm_ref and abs(factor - exp_factor) < 1e-5
        pn, _, _ = orc.adamw_step(params, g_ref * np.float32(exp_factor), np.zeros_like(params), np.zeros_like(params), 1e-2, 0.9, 0.95, 1e-8, 0.1, 1)
        expect = np.where(mask, pn, params)
        assert rel(model.read_params(), expect) < 1e-5
        model.close()


def test_shape_errors_are_reported_not_ignored(ctx):
    cfg = oracle.Config(**TOY)
    model = bridge.Model(ctx, cfg, "f32")
    tok = np.zeros((cfg.B, cfg.S * 2), np.int32)
    with pytest.raises(bridge.B200Error):          # longer than max_seq_len (cpp/src/Positional.cpp:90-94)
        model.train_step_host(tok, tok)
    bad = np.full((cfg.B, cfg.S), cfg.V + 5, np.int32)
    with pytest.raises(bridge.B200Error):          # token id out of range (cpp/src/Transformer.cpp:127-129)
        model.loss_and_grads_host(bad, np.zeros_like(bad))
    model.close()
