"""Tensor-core causal GQA attention (bf16, head_dim 64/128) forward and backward against the CPU
checker on bf16-rounded inputs (rel-err <= 2e-2): group sizes 1/2/4, ragged sequence lengths, and the
attention benchmark configuration (B8 S2048 16q/4kv hd128) checked on EVERY (batch, kv-group) slice for the
default kernels (L2 ratio and largest element error), one slice for the alternative forms, plus
size-independent properties (causality, linearity of the backward in dO)."""
import numpy as np
import pytest

from gpu_util import BF16_TOL, bridge, ctx, rel, synth  # noqa: F401

pytestmark = pytest.mark.gpu
SEED = 31


@pytest.fixture(params=[1, 0], ids=["second_forms", "first_forms"], autouse=True)
def kernel_choice(ctx, request):
    """Every test runs with both forms of the forward and of the backward kernel (internal A/B hooks of the library)."""
    default_bwd2 = 1
    for name in ("b200_internal_set_attn_fwd2", "b200_internal_set_attn_bwd2"):
        getattr(ctx.lib, name).argtypes = [bridge._vp, bridge._i]
    ctx.lib.b200_internal_set_attn_fwd2(ctx.h, request.param)
    ctx.lib.b200_internal_set_attn_bwd2(ctx.h, request.param)
    yield
    ctx.lib.b200_internal_set_attn_fwd2(ctx.h, 1)
    ctx.lib.b200_internal_set_attn_bwd2(ctx.h, default_bwd2)


def make(B, nH, nKV, S, hd, seed=SEED):
    q = synth.bf16_round(synth.normal(seed, "q", (B, nH, S, hd)))
    k = synth.bf16_round(synth.normal(seed, "k", (B, nKV, S, hd)))
    v = synth.bf16_round(synth.normal(seed, "v", (B, nKV, S, hd)))
    dO = synth.bf16_round(synth.normal(seed, "dO", (B, S, nH * hd)))
    return q, k, v, dO


@pytest.mark.parametrize("B,nH,nKV,S,hd", [(1, 1, 1, 128, 128), (1, 2, 1, 256, 128), (2, 4, 2, 384, 128),
                                           (1, 4, 1, 200, 128), (2, 4, 4, 72, 64), (1, 8, 2, 520, 64), (1, 2, 2, 1, 128),
                                           # odd numbers of 64-query steps per key tile, a lone step, a ragged last step
                                           (1, 1, 1, 192, 128), (1, 3, 3, 64, 128), (2, 2, 2, 320, 128), (1, 3, 1, 84, 128)])
def test_forward_and_backward_match_the_checker(ctx, orc, B, nH, nKV, S, hd):
    q, k, v, dO = make(B, nH, nKV, S, hd)
    dq_, dk_, dv_ = ctx.array(q, "bf16"), ctx.array(k, "bf16"), ctx.array(v, "bf16")
    o, lse = ctx.flash_attn_fwd(dq_, dk_, dv_, want_lse=True)
    eo = orc.attention_forward(q, k, v)
    assert rel(o.download(), eo) < BF16_TOL
    scale = 1 / np.sqrt(hd)
    s00 = (q[0, 0].astype(np.float64) @ k[0, 0].astype(np.float64).T) * scale
    s00 = np.where(np.tril(np.ones((S, S), bool)), s00, -np.inf)
    np.testing.assert_allclose(lse.download()[0, 0], np.log(np.exp(s00 - s00.max(-1, keepdims=True)).sum(-1)) + s00.max(-1), rtol=2e-3, atol=2e-3)
    gq, gk, gv = ctx.fused_attn_bwd(dq_, dk_, dv_, ctx.array(dO, "bf16"))
    eq, ek, ev = orc.attention_backward(q, k, v, dO)
    if S == 1:      # a single key: P == 1 and dS == 0 exactly, so dQ and dK vanish
        assert np.abs(gq.download()).max() < 1e-5 and np.abs(gk.download()).max() < 1e-5
    else:
        assert rel(gq.download(), eq) < BF16_TOL, "dQ"
        assert rel(gk.download(), ek) < BF16_TOL, "dK"
    assert rel(gv.download(), ev) < BF16_TOL, "dV"


def maxerr(a, e):
    """Largest element error relative to the largest reference element: one wrong tile shows here even where the
    L2 ratio over a large array would hide it."""
    return float(np.abs(np.asarray(a, np.float64) - e).max() / (np.abs(e).max() + 1e-30))


def test_benchmark_configuration_slice_and_properties(ctx, orc, request):
    B, nH, nKV, S, hd = 8, 16, 4, 2048, 128
    G = nH // nKV
    q = ctx.empty((B, nH, S, hd), "bf16"); k = ctx.empty((B, nKV, S, hd), "bf16"); v = ctx.empty((B, nKV, S, hd), "bf16")
    dO = ctx.empty((B, S, nH * hd), "bf16")
    for a, sd in ((q, 1), (k, 2), (v, 3), (dO, 4)):
        ctx._check(ctx.lib.b200_fill_normal(ctx.h, a.ptr, 1, a.size, sd, 1.0))
    o, lse = ctx.flash_attn_fwd(q, k, v, want_lse=True)
    gq, gk, gv = ctx.fused_attn_bwd(q, k, v, dO)
    hq, hk, hv, hdO = q.download(), k.download(), v.download(), dO.download()
    ho, hgq, hgk, hgv = o.download(), gq.download(), gk.download(), gv.download()
    # the backward that takes the forward's saved output and log-sum-exp gives the same gradients as the one that recomputes them
    sq_, sk_, sv_ = ctx.flash_attn_bwd(q, k, v, o, dO, lse)
    assert rel(sq_.download(), hgq) < 1e-3 and rel(sk_.download(), hgk) < 1e-3 and rel(sv_.download(), hgv) < 1e-3
    # the default kernels: EVERY (batch, KV head) slice of the benchmark shape against the checker; the other forms: one slice
    second_forms = "second_forms" in request.node.name
    slices = [(b, kvh) for b in range(B) for kvh in range(nKV)] if second_forms else [(5, 2)]
    for b, kvh in slices:
        sq = hq[b:b + 1, kvh * G:(kvh + 1) * G]; sk = hk[b:b + 1, kvh:kvh + 1]; sv = hv[b:b + 1, kvh:kvh + 1]
        sdO = np.ascontiguousarray(hdO[b:b + 1, :, kvh * G * hd:(kvh + 1) * G * hd])
        eo = orc.attention_forward(sq, sk, sv)
        go = ho[b:b + 1, :, kvh * G * hd:(kvh + 1) * G * hd]
        assert rel(go, eo) < BF16_TOL and maxerr(go, eo) < BF16_TOL, (b, kvh)
        eq, ek, ev = orc.attention_backward(sq, sk, sv, sdO)
        for name, got, exp in (("dQ", hgq[b:b + 1, kvh * G:(kvh + 1) * G], eq), ("dK", hgk[b:b + 1, kvh:kvh + 1], ek),
                               ("dV", hgv[b:b + 1, kvh:kvh + 1], ev)):
            assert rel(got, exp) < BF16_TOL and maxerr(got, exp) < 2 * BF16_TOL, (name, b, kvh, rel(got, exp), maxerr(got, exp))
    # causality at full size: changing keys/values from position 1500 on leaves earlier outputs bit-identical
    hk2, hv2 = hk.copy(), hv.copy()
    hk2[:, :, 1500:] *= -1.0
    hv2[:, :, 1500:] += 1.0
    o2 = ctx.flash_attn_fwd(q, ctx.array(hk2, "bf16"), ctx.array(hv2, "bf16")).download()
    np.testing.assert_array_equal(o2[:, :1500], ho[:, :1500])
    assert np.isfinite(ho).all()
    # the backward is linear in dO: doubling dO doubles dV exactly (powers of two are exact in bf16)
    gq2, gk2, gv2 = ctx.fused_attn_bwd(q, k, v, ctx.array(2.0 * hdO, "bf16"))
    np.testing.assert_array_equal(gv2.download(), 2.0 * gv.download())
