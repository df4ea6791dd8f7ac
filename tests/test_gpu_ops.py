"""GPU parity of every op of the decoder-block path against the CPU checker, through the
C ABI, on seeded inputs.  fp32: rel-err <= 1e-4; bf16: rel-err <= 2e-2 against the fp32
checker run on the bf16-rounded inputs.  Edge cases follow the reference's tests: ragged
and empty shapes, large-magnitude logits, causal masking, GQA group sizes 1/2/4."""
import numpy as np
import pytest

from gpu_util import BF16_TOL, FP32_TOL, bridge, ctx, rel, synth  # noqa: F401

pytestmark = pytest.mark.gpu
SEED = 77


def _in(a, dtype):
    return synth.bf16_round(a) if dtype == "bf16" else a


def _tol(dtype):
    return BF16_TOL if dtype == "bf16" else FP32_TOL


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("rows,D", [(6, 32), (37, 256), (5, 2048), (3, 100), (2, 8200)])
def test_rms_norm_forward_backward(ctx, orc, dtype, rows, D):
    x = _in(synth.normal(SEED, "x", (rows, D)), dtype)
    w = _in(1.0 + 0.1 * synth.normal(SEED, "w", (D,)), dtype)
    g = _in(synth.normal(SEED, "g", (rows, D)), dtype)
    dx_, dw_, dg_ = ctx.array(x, dtype), ctx.array(w, dtype), ctx.array(g, dtype)
    y, rstd = ctx.rms_norm_forward(dx_, dw_, want_rstd=True)
    assert rel(y.download(), orc.rms_norm_forward(x, w)) < _tol(dtype)
    np.testing.assert_allclose(rstd.download(), 1 / np.sqrt((x.astype(np.float64) ** 2).mean(-1) + 1e-5), rtol=1e-5)
    gx, gw = ctx.rms_norm_backward(dg_, dx_, dw_)
    ex, ew = orc.rms_norm_backward(g, x, w)
    assert rel(gx.download(), ex) < _tol(dtype)
    assert rel(gw.download(), ew) < 1e-4


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_fused_add_norm_and_its_backward(ctx, orc, dtype):
    rows, D = 19, 256
    h = _in(synth.normal(SEED, "h", (rows, D)), dtype)
    r = _in(synth.normal(SEED, "r", (rows, D)), dtype)
    w = _in(1.0 + 0.1 * synth.normal(SEED, "w", (D,)), dtype)
    dh = ctx.array(h, dtype)
    out = ctx.fused_add_norm(dh, ctx.array(r, dtype), ctx.array(w, dtype))
    hsum = _in(h + r, dtype)
    assert rel(dh.download(), h + r) < _tol(dtype)                      # h += r, in place
    assert rel(out.download(), orc.rms_norm_forward(hsum, w)) < _tol(dtype)
    g = _in(synth.normal(SEED, "g", (rows, D)), dtype)
    rg = _in(synth.normal(SEED, "rg", (rows, D)), dtype)
    dx = ctx.fused_backward_add_norm(ctx.array(g, dtype), ctx.array(h, dtype), ctx.array(w, dtype), ctx.array(rg, dtype))
    ex, _ = orc.rms_norm_backward(g, h, w, want_dw=False)
    assert rel(dx.download(), ex + rg) < _tol(dtype)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("hd", [4, 8, 32, 128])
def test_rope_tables_forward_backward(ctx, orc, dtype, hd):
    B, qh, kvh, S = 2, 4, 2, 24
    c, s = ctx.rope_tables(S, hd)
    ec, es = orc.rope_tables(S, hd)
    np.testing.assert_allclose(c.download(), ec, atol=2e-6)
    np.testing.assert_allclose(s.download(), es, atol=2e-6)
    q = _in(synth.normal(SEED, "q", (B, qh, S, hd)), dtype)
    k = _in(synth.normal(SEED, "k", (B, kvh, S, hd)), dtype)
    dq, dk = ctx.array(q, dtype), ctx.array(k, dtype)
    ctx.rope_forward(dq, dk, c, s)
    assert rel(dq.download(), orc.rope(q, ec, es)) < _tol(dtype)
    assert rel(dk.download(), orc.rope(k, ec, es)) < _tol(dtype)
    dg = ctx.array(q, dtype)
    ctx.rope_backward(dg, c, s)
    assert rel(dg.download(), orc.rope(q, ec, es, backward=True)) < _tol(dtype)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("n", [200, 4096 * 3, 7])
def test_swiglu_and_residual_add(ctx, orc, dtype, n):
    gate, up, dy = (_in(synth.normal(SEED, nm, (n,)), dtype) for nm in ("gate", "up", "dy"))
    dg_, du_, dy_ = ctx.array(gate, dtype), ctx.array(up, dtype), ctx.array(dy, dtype)
    assert rel(ctx.swiglu_forward(dg_, du_).download(), orc.swiglu_forward(gate, up)) < _tol(dtype)
    gg, gu = ctx.swiglu_backward(dy_, dg_, du_)
    eg, eu = orc.swiglu_backward(dy, gate, up)
    assert rel(gg.download(), eg) < _tol(dtype) and rel(gu.download(), eu) < _tol(dtype)
    ctx.residual_add(dg_, du_)
    assert rel(dg_.download(), gate + up) < _tol(dtype)


def test_swiglu_known_answers(ctx):
    # cpp/tests/test_activations.cpp:48-75
    y = ctx.swiglu_forward(ctx.array(np.array([0.0, 2.0], np.float32)), ctx.array(np.array([10.0, 5.0], np.float32)))
    np.testing.assert_allclose(y.download(), [0.0, 8.80797], atol=1e-5)


def test_rmsnorm_known_answers(ctx):
    # cpp/tests/test_rmsnorm.cpp:49,75-78
    x = np.array([[0.3, 0.9], [-0.7, 0.4]], np.float32)
    y = ctx.rms_norm_forward(ctx.array(x), ctx.array(np.ones(2, np.float32)))
    np.testing.assert_allclose(y.download().ravel(), [0.447208, 1.341625, -1.22786, 0.701635], atol=2e-5)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_head_split_and_merge_round_trip(ctx, orc, dtype):
    B, n, S, hd = 2, 3, 5, 8
    x = _in(synth.normal(SEED, "x3", (B, S, n * hd)), dtype)
    d4 = ctx.reshape_to_4d(ctx.array(x, dtype), B, n, S, hd)
    exp = x.reshape(B, S, n, hd).transpose(0, 2, 1, 3)
    np.testing.assert_array_equal(d4.download(), exp)
    np.testing.assert_array_equal(ctx.reshape_to_3d(d4, B, n, S, hd).download(), x)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_embedding_gather_and_scatter(ctx, dtype):
    V, H, T = 50, 64, 40
    table = _in(synth.normal(SEED, "table", (V, H), 0.02), dtype)
    ids = synth.token_ids(SEED, "ids", (T,), V)
    ids[:4] = ids[4]                                  # collisions
    dids = ctx.array(ids.astype(np.uint32), "u32")
    out = ctx.embedding_forward(dids, ctx.array(table, dtype))
    np.testing.assert_array_equal(out.download(), table[ids])
    gh = _in(synth.normal(SEED, "gh", (T, H)), dtype)
    gt = ctx.embedding_backward(dids, ctx.array(gh, dtype), V).download()
    exp = np.zeros((V, H), np.float64)
    np.add.at(exp, ids, gh.astype(np.float64))
    assert rel(gt, exp) < 1e-6


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("T,V", [(10, 50), (33, 4096), (4, 32000), (5, 1001)])
def test_cross_entropy(ctx, orc, dtype, T, V):
    lg = _in(synth.normal(SEED, "logits", (T, V), 3.0), dtype)
    tg = synth.token_ids(SEED, "tg", (T,), V)
    loss, grad = ctx.cross_entropy(ctx.array(lg, dtype), ctx.array(tg.astype(np.uint32), "u32"))
    el, eg = orc.cross_entropy(lg, tg)
    assert abs(float(loss.download()[0]) - el) < 1e-5 * max(1, abs(el))
    assert rel(grad.download(), eg) < _tol(dtype)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("T,V", [(64, 4096), (7, 1001), (300, 32000)])
def test_cross_entropy_in_place_matches_out_of_place(ctx, dtype, T, V):
    # the engine's calling form: the gradient overwrites the logits (allowed by the header)
    lg = _in(synth.normal(SEED, "logits_ip", (T, V), 3.0), dtype)
    tg = ctx.array(synth.token_ids(SEED, "tg_ip", (T,), V).astype(np.uint32), "u32")
    loss, grad = ctx.cross_entropy(ctx.array(lg, dtype), tg)
    buf = ctx.array(lg, dtype)
    for _ in range(3):          # a stale read of an already overwritten target logit would change the loss
        buf.upload(lg)
        loss_ip, grad_ip = ctx.cross_entropy(buf, tg, in_place=True)
        assert float(loss_ip.download()[0]) == float(loss.download()[0])
        np.testing.assert_array_equal(grad_ip.download(), grad.download())


def test_cross_entropy_known_answers(ctx):
    # cpp/tests/test_loss.cpp:56-101
    loss, grad = ctx.cross_entropy(ctx.array(np.zeros((1, 4), np.float32)), ctx.array(np.array([2], np.uint32), "u32"))
    assert abs(float(loss.download()[0]) - np.log(4.0)) < 1e-5
    np.testing.assert_allclose(grad.download()[0], [0.25, 0.25, -0.75, 0.25], atol=1e-6)
    loss, _ = ctx.cross_entropy(ctx.array(np.full((1, 4), 1000.0, np.float32)), ctx.array(np.array([1], np.uint32), "u32"))
    assert np.isfinite(loss.download()[0]) and abs(float(loss.download()[0]) - np.log(4.0)) < 1e-5


@pytest.mark.parametrize("shadow", [False, True])
def test_adamw_step(ctx, orc, shadow):
    n = 1003
    p, g = synth.normal(SEED, "p", (n,), 0.02), synth.normal(SEED, "g", (n,), 0.01)
    m0, v0 = 0.001 * synth.normal(SEED, "m", (n,)), np.abs(1e-5 * synth.normal(SEED, "v", (n,)))
    dp, dm, dv = ctx.array(p), ctx.array(m0), ctx.array(v0)
    sh = ctx.empty((n,), "bf16") if shadow else None
    ctx.adamw_step(dp, ctx.array(g), dm, dv, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3, shadow=sh)
    ep, em, ev = orc.adamw_step(p, g, m0, v0, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3)
    assert rel(dp.download(), ep) < 1e-6 and rel(dm.download(), em) < 1e-6 and rel(dv.download(), ev) < 1e-6
    if shadow:
        np.testing.assert_array_equal(sh.download(), synth.bf16_round(dp.download()))


@pytest.mark.parametrize("M,N,K", [(2, 2, 3), (7, 5, 9), (256, 256, 256), (256, 688, 256), (130, 70, 33), (256, 4096, 256)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_fp32(ctx, orc, M, N, K, ta, tb):
    A = synth.normal(SEED, "A", (K, M) if ta else (M, K))
    B = synth.normal(SEED, "B", (N, K) if tb else (K, N))
    out = ctx.gemm(ctx.array(A), ctx.array(B), M, N, K, ta, tb).download()
    assert rel(out, orc.gemm(A, B, M, N, K, ta, tb)) < 1e-5
    if (M, N, K) == (7, 5, 9):      # accumulate into C
        C0 = synth.normal(SEED, "C0", (M, N))
        dc = ctx.array(C0)
        ctx.gemm(ctx.array(A), ctx.array(B), M, N, K, ta, tb, C_acc=dc)
        assert rel(dc.download(), orc.gemm(A, B, M, N, K, ta, tb, C_in=C0)) < 1e-5


def test_matmul_known_answers(ctx):
    # cpp/tests/test_math_ops.cpp:167-188
    A = np.arange(1, 7, dtype=np.float32).reshape(2, 3)
    B = np.arange(7, 13, dtype=np.float32).reshape(3, 2)
    np.testing.assert_array_equal(ctx.gemm(ctx.array(A), ctx.array(B), 2, 2, 3).download(), [[58, 64], [139, 154]])


@pytest.mark.parametrize("B,nH,nKV,S,hd", [(1, 4, 2, 6, 4), (2, 8, 2, 128, 32), (2, 4, 4, 33, 16), (1, 4, 1, 70, 64), (1, 2, 1, 40, 128)])
def test_attention_fp32_forward_backward(ctx, orc, B, nH, nKV, S, hd):
    q = synth.normal(SEED, "q", (B, nH, S, hd))
    k = synth.normal(SEED, "k", (B, nKV, S, hd))
    v = synth.normal(SEED, "v", (B, nKV, S, hd))
    dO = synth.normal(SEED, "dO", (B, S, nH * hd))
    dq_, dk_, dv_ = ctx.array(q), ctx.array(k), ctx.array(v)
    o, lse = ctx.flash_attn_fwd(dq_, dk_, dv_, want_lse=True)
    assert rel(o.download(), orc.attention_forward(q, k, v)) < FP32_TOL
    gq, gk, gv = ctx.fused_attn_bwd(dq_, dk_, dv_, ctx.array(dO))
    eq, ek, ev = orc.attention_backward(q, k, v, dO)
    assert rel(gq.download(), eq) < FP32_TOL and rel(gk.download(), ek) < FP32_TOL and rel(gv.download(), ev) < FP32_TOL


def test_attention_is_causal_and_handles_extreme_inputs(ctx):
    # cpp/tests/test_attention.cpp:99-115 (mask leak) and the overflow/underflow cases
    B, nH, nKV, S, hd = 1, 4, 2, 16, 8
    q, k, v = (synth.normal(SEED, n, (B, h, S, hd)) for n, h in (("q", nH), ("k", nKV), ("v", nKV)))
    base = ctx.flash_attn_fwd(ctx.array(q), ctx.array(k), ctx.array(v)).download()
    k2, v2 = k.copy(), v.copy()
    k2[:, :, 10:] += 7.0
    v2[:, :, 10:] -= 3.0
    moved = ctx.flash_attn_fwd(ctx.array(q), ctx.array(k2), ctx.array(v2)).download()
    np.testing.assert_array_equal(moved[:, :10], base[:, :10])
    big = ctx.flash_attn_fwd(ctx.array(q * 1e4), ctx.array(k * 1e4), ctx.array(v)).download()
    assert np.isfinite(big).all()
    zero = ctx.flash_attn_fwd(ctx.array(q * 0), ctx.array(k * 0), ctx.array(v * 0)).download()
    assert not zero.any()


def test_empty_inputs_are_no_ops(ctx):
    e = ctx.empty((0,), "f32")
    ctx.residual_add(e, e)
    ctx.swiglu_forward(e, e)
    ctx.sync()


def test_host_pointer_calls_follow_the_reference_convention(ctx, orc):
    A, B = synth.normal(SEED, "hA", (33, 17)), synth.normal(SEED, "hB", (17, 29))
    assert rel(ctx.host_gemm(A, B, 33, 29, 17), orc.gemm(A, B, 33, 29, 17)) < 1e-5
    x, w = synth.normal(SEED, "hx", (9, 64)), np.ones(64, np.float32)
    assert rel(ctx.host_rms_norm_forward(x, w), orc.rms_norm_forward(x, w)) < 1e-5
    q, k, v = (synth.normal(SEED, n, (1, h, 20, 16)) for n, h in (("hq", 4), ("hk", 2), ("hv", 2)))
    assert rel(ctx.host_flash_attn_fwd(q, k, v), orc.attention_forward(q, k, v)) < FP32_TOL
    dO = synth.normal(SEED, "hdO", (1, 20, 64))
    got, exp = ctx.host_fused_attn_bwd(q, k, v, dO), orc.attention_backward(q, k, v, dO)
    assert all(rel(a, b) < FP32_TOL for a, b in zip(got, exp))
    lg, tg = synth.normal(SEED, "hl", (6, 40), 2.0), synth.token_ids(SEED, "ht", (6,), 40)
    loss, grad = ctx.host_cross_entropy(lg, tg)
    el, eg = orc.cross_entropy(lg, tg)
    assert abs(loss - el) < 1e-5 and rel(grad, eg) < 1e-5
