"""Vocabulary projection fused with cross-entropy (b200_vocab_ce_forward / _backward) against the CPU
checker: loss, log-sum-exp, logits gradient, dW and dx -- with the logits never stored (statistics in the
GEMM epilogue, gradient by a second run of the projection) and with stored logits converted in place;
fp32 on the CUDA cores; ragged shapes; the reference's known answers for the loss; and the 1.6B
configuration's full [16384, 2048] x [2048, 32000] shape on sampled rows (the checker recomputes those rows)."""
import numpy as np
import pytest

from gpu_util import BF16_TOL, FP32_TOL, bridge, ctx, rel, synth  # noqa: F401

pytestmark = pytest.mark.gpu
SEED = 77


def _case(T, H, V, dtype, std_w=0.05):
    x = synth.normal(SEED, f"x{T}", (T, H))
    w = synth.normal(SEED, f"w{V}", (H, V), std_w)
    if dtype == "bf16":
        x, w = synth.bf16_round(x), synth.bf16_round(w)
    tg = synth.token_ids(SEED, f"t{T}", (T,), V)
    return x, w, tg


def _expected(orc, x, w, tg):
    T, H = x.shape
    V = w.shape[1]
    logits = orc.gemm(x, w, T, V, H)
    loss, dl = orc.cross_entropy(logits, tg)
    lse = np.log(np.exp(logits.astype(np.float64) - logits.max(1, keepdims=True)).sum(1)) + logits.max(1)
    return loss, lse, dl, orc.gemm(x, dl, H, V, T, transA=True), orc.gemm(dl, w, T, H, V, transB=True)


@pytest.mark.parametrize("keep_logits", [False, True], ids=["logits_never_stored", "logits_stored_then_converted"])
@pytest.mark.parametrize("T,H,V", [(256, 128, 512), (300, 64, 1000), (1000, 256, 2056), (37, 72, 264), (2048, 256, 4096)])
def test_bf16_forward_and_backward(ctx, orc, T, H, V, keep_logits):
    x, w, tg = _case(T, H, V, "bf16")
    loss_e, lse_e, dl_e, gw_e, gx_e = _expected(orc, x, w, tg)
    dx, dw, dt = ctx.array(x, "bf16"), ctx.array(w, "bf16"), ctx.array(tg.astype(np.uint32), "u32")
    out = ctx.vocab_ce_forward(dx, dw, dt, want_logits=keep_logits)
    loss, lse = float(out[0].download()[0]), out[1].download()
    tol = 2e-3 if keep_logits else 1e-5          # stored logits are rounded to bf16 before the statistics
    assert abs(loss - loss_e) < tol * max(1.0, abs(loss_e)), (loss, loss_e)
    assert np.abs(lse - lse_e).max() < (2e-2 if keep_logits else 1e-4)
    if keep_logits:
        assert rel(out[2].download(), orc.gemm(x, w, T, V, H)) < 5e-3
    dl, gw, gx = ctx.vocab_ce_backward(dx, dw, dt, out[1], logits=out[2] if keep_logits else None)
    assert rel(dl.download(), dl_e) < BF16_TOL
    assert rel(gw.download(), gw_e) < BF16_TOL and rel(gx.download(), gx_e) < BF16_TOL
    assert np.abs(gw.download() - gw_e).max() < BF16_TOL * np.abs(gw_e).max() * 4


@pytest.mark.parametrize("T,H,V", [(64, 32, 100), (256, 256, 4096), (10, 16, 50)])
def test_fp32_forward_and_backward(ctx, orc, T, H, V):
    x, w, tg = _case(T, H, V, "f32")
    loss_e, lse_e, dl_e, gw_e, gx_e = _expected(orc, x, w, tg)
    dx, dw, dt = ctx.array(x), ctx.array(w), ctx.array(tg.astype(np.uint32), "u32")
    loss, lse, logits = ctx.vocab_ce_forward(dx, dw, dt, want_logits=True)
    assert abs(float(loss.download()[0]) - loss_e) < 1e-5 * max(1.0, abs(loss_e))
    assert np.abs(lse.download() - lse_e).max() < 1e-4
    dl, gw, gx = ctx.vocab_ce_backward(dx, dw, dt, lse, logits=logits)
    assert rel(dl.download(), dl_e) < FP32_TOL and rel(gw.download(), gw_e) < FP32_TOL and rel(gx.download(), gx_e) < FP32_TOL
    loss2, lse2 = ctx.vocab_ce_forward(dx, dw, dt)              # logits in the context workspace
    assert float(loss2.download()[0]) == float(loss.download()[0])
    dl2, _, _ = ctx.vocab_ce_backward(dx, dw, dt, lse2)          # projection run again
    assert rel(dl2.download(), dl_e) < FP32_TOL


def test_known_answers_of_the_reference_loss_tests(ctx):
    # cpp/tests/test_loss.cpp:56-101: uniform logits -> log(V); a dominant logit -> ~0 loss, finite for huge values
    H, V, T = 64, 512, 256
    x = np.zeros((T, H), np.float32)
    w = synth.bf16_round(synth.normal(SEED, "wk", (H, V), 0.05))
    tg = synth.token_ids(SEED, "tk", (T,), V).astype(np.uint32)
    loss, lse = ctx.vocab_ce_forward(ctx.array(x, "bf16"), ctx.array(w, "bf16"), ctx.array(tg, "u32"))
    assert abs(float(loss.download()[0]) - np.log(V)) < 1e-5
    x[:, 0] = 1.0
    w2 = np.zeros((H, V), np.float32)
    w2[0, :] = -200.0
    w2[0, 5] = 200.0
    loss, lse = ctx.vocab_ce_forward(ctx.array(x, "bf16"), ctx.array(w2, "bf16"), ctx.array(np.full(T, 5, np.uint32), "u32"))
    assert abs(float(loss.download()[0])) < 1e-5
    loss, _ = ctx.vocab_ce_forward(ctx.array(x, "bf16"), ctx.array(w2, "bf16"), ctx.array(np.full(T, 6, np.uint32), "u32"))
    assert abs(float(loss.download()[0]) - 34.538776) < 1e-3        # probability clamped at 1e-15 (cpp/src/Loss.cpp:113-117)


def test_full_vocabulary_projection_shape_on_sampled_rows(ctx, orc):
    T, H, V = 16384, 2048, 32000
    x = synth.bf16_round(synth.normal(SEED, "xf", (T, H)))
    dw_ = ctx.empty((H, V), "bf16")
    ctx._check(ctx.lib.b200_fill_normal(ctx.h, dw_.ptr, bridge.BF16, H * V, 99, 0.02))
    w = dw_.download()
    tg = synth.token_ids(SEED, "tf", (T,), V)
    dx, dt = ctx.array(x, "bf16"), ctx.array(tg.astype(np.uint32), "u32")
    loss, lse = ctx.vocab_ce_forward(dx, dw_, dt)
    rows = np.concatenate([[0, 127, 128, 255, 256, T - 1], np.random.default_rng(3).integers(0, T, 58)])
    lg = x[rows].astype(np.float64) @ w.astype(np.float64)
    lse_e = np.log(np.exp(lg - lg.max(1, keepdims=True)).sum(1)) + lg.max(1)
    assert np.abs(lse.download()[rows] - lse_e).max() < 1e-4
    # every row's loss is lse - target logit; the mean over all rows must equal the reported loss
    tl = np.einsum("th,ht->t", x.astype(np.float64), w[:, tg].astype(np.float64))
    assert abs(float(loss.download()[0]) - float(np.mean(lse.download().astype(np.float64) - tl))) < 1e-5
    dl, gw, gx = ctx.vocab_ce_backward(dx, dw_, dt, lse)
    p = np.exp(lg - lse_e[:, None])
    p[np.arange(len(rows)), tg[rows]] -= 1.0
    dl_h = dl.download()                                   # [16384, 32000] once
    got = dl_h[rows]
    assert rel(got, p / T) < BF16_TOL
    assert np.abs(got - p / T).max() < 2e-2 * np.abs(p / T).max()
    # the gradient of a softmax sums to zero over the vocabulary: every row, without the checker
    assert np.abs(dl_h.sum(1, dtype=np.float64)).max() < 1e-5
    # dx on the sampled rows from the checker's gradient; dW through linearity on sampled columns
    assert rel(gx.download()[rows], (p / T) @ w.astype(np.float64).T) < BF16_TOL
    cols = np.random.default_rng(4).integers(0, V, 48)
    dl_cols = dl_h[:, cols].astype(np.float64)
    assert rel(gw.download()[:, cols], x.astype(np.float64).T @ dl_cols) < 1e-3
