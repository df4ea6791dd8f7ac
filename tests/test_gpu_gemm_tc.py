"""The tcgen05 bf16 GEMM (NN forward, NT data-gradient, TN weight-gradient forms) against the
CPU checker on bf16-rounded inputs, bf16 and fp32 outputs, ragged edges, accumulate; then the
full projection shapes of the 1.6B configuration through a size-independent property
(sampled rows/columns recomputed on the CPU, and linearity in A)."""
import numpy as np
import pytest

from gpu_util import BF16_TOL, bridge, ctx, rel, synth  # noqa: F401

pytestmark = pytest.mark.gpu
SEED = 5


def _ab(M, N, K, ta, tb, std_b=1.0):
    A = synth.bf16_round(synth.normal(SEED, f"A{M}{K}", (K, M) if ta else (M, K)))
    B = synth.bf16_round(synth.normal(SEED, f"B{K}{N}", (N, K) if tb else (K, N), std_b))
    return A, B


def _ref(A, B, ta, tb):
    a = A.T if ta else A
    b = B.T if tb else B
    return a.astype(np.float64) @ b.astype(np.float64)


FORMS = [(False, False), (False, True), (True, False), (True, True)]


@pytest.fixture(params=[1, 0], ids=["two_cta", "one_cta"], autouse=True)
def gemm_kernel_choice(ctx, request):
    """Every test runs with the two-CTA (cta_group::2) kernel enabled for large shapes and with the
    single-CTA kernel forced (internal A/B hook of the library)."""
    ctx.lib.b200_internal_set_gemm_2cta.argtypes = [bridge._vp, bridge._i]
    ctx.lib.b200_internal_set_gemm_2cta(ctx.h, request.param)
    yield
    ctx.lib.b200_internal_set_gemm_2cta(ctx.h, 1)


@pytest.mark.parametrize("ta,tb", FORMS)
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (384, 256, 1024)])
def test_aligned_tiles(ctx, ta, tb, M, N, K):
    A, B = _ab(M, N, K, ta, tb)
    exp = _ref(A, B, ta, tb)
    out32 = ctx.gemm(ctx.array(A, "bf16"), ctx.array(B, "bf16"), M, N, K, ta, tb, out_dtype="f32").download()
    assert rel(out32, exp) < 1e-5, "fp32-out tensor-core GEMM must be exact up to accumulation order"
    out16 = ctx.gemm(ctx.array(A, "bf16"), ctx.array(B, "bf16"), M, N, K, ta, tb, out_dtype="bf16").download()
    assert rel(out16, exp) < 5e-3


@pytest.mark.parametrize("ta,tb", FORMS)
@pytest.mark.parametrize("M,N,K", [(8, 8, 8), (136, 264, 72), (200, 328, 200), (1000, 520, 136), (16, 3072, 2048), (2500, 2200, 200), (3000, 9000, 72)])
def test_ragged_edges(ctx, ta, tb, M, N, K):
    A, B = _ab(M, N, K, ta, tb)
    out = ctx.gemm(ctx.array(A, "bf16"), ctx.array(B, "bf16"), M, N, K, ta, tb, out_dtype="f32").download()
    assert rel(out, _ref(A, B, ta, tb)) < 1e-5


def test_accumulate_into_fp32_c(ctx):
    M, N, K = 256, 512, 192
    A, B = _ab(M, N, K, True, False)
    C0 = synth.normal(SEED, "C0", (M, N))
    dc = ctx.array(C0)
    ctx.gemm(ctx.array(A, "bf16"), ctx.array(B, "bf16"), M, N, K, True, False, C_acc=dc)
    assert rel(dc.download(), _ref(A, B, True, False) + C0) < 1e-5


@pytest.mark.parametrize("M,N,K,acc", [(1024, 1280, 8192, False), (1000, 1300, 8200, False), (2048, 2048, 16384, False), (512, 2304, 12288, True)])
def test_weight_gradient_shapes_whole_result(ctx, M, N, K, acc):
    """Few tiles and a deep K (the weight-gradient form, fp32 result, split K where the tiles fill the GPU badly; partial
    tiles are added with reductions): the whole result against the float64 product."""
    A, B = _ab(M, N, K, True, False, std_b=0.05)
    exp = _ref(A, B, True, False)
    da, db = ctx.array(A, "bf16"), ctx.array(B, "bf16")
    if acc:
        C0 = synth.normal(SEED, "C0s", (M, N))
        dc = ctx.array(C0)
        ctx.gemm(da, db, M, N, K, True, False, C_acc=dc)
        got, exp = dc.download(), exp + C0
    else:
        got = ctx.gemm(da, db, M, N, K, True, False, out_dtype="f32").download()
    assert rel(got, exp) < 2.5e-5              # fp32 accumulation over up to 16384 products
    assert np.abs(got - exp).max() < 2e-4 * np.abs(exp).max()


def test_many_tiles_exercise_the_persistent_schedule(ctx):
    M, N, K = 128 * 21, 256 * 9, 320          # 189 tiles > 148 SMs, odd counts
    A, B = _ab(M, N, K, False, False)
    out = ctx.gemm(ctx.array(A, "bf16"), ctx.array(B, "bf16"), M, N, K, out_dtype="f32").download()
    assert rel(out, _ref(A, B, False, False)) < 1e-5


@pytest.mark.parametrize("M", [1, 7, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(8, 8), (104, 72), (2048, 2048), (3072, 2048), (11264, 2048), (2048, 5632), (32000, 2048), (200, 4096)])
def test_few_row_weight_streaming_kernel(ctx, M, N, K):
    """Decode-shaped GEMMs (rows = sequences) go through the swapped-operand, cluster split-K kernel:
    exact against the CPU product up to accumulation order, bit-identical between runs, and equal to the
    general tile kernel within rounding."""
    A, B = _ab(M, N, K, False, False, std_b=0.05)
    exp = _ref(A, B, False, False)
    da, db = ctx.array(A, "bf16"), ctx.array(B, "bf16")
    out32 = ctx.gemm(da, db, M, N, K, out_dtype="f32").download()
    assert rel(out32, exp) < 1e-5
    np.testing.assert_array_equal(out32, ctx.gemm(da, db, M, N, K, out_dtype="f32").download())
    out16 = ctx.gemm(da, db, M, N, K, out_dtype="bf16").download()
    assert rel(out16, exp) < 5e-3
    ctx.lib.b200_internal_set_gemm_skinny.argtypes = [bridge._vp, bridge._i]
    ctx.lib.b200_internal_set_gemm_skinny(ctx.h, 0)
    try:
        tile = ctx.gemm(da, db, M, N, K, out_dtype="f32").download()
    finally:
        ctx.lib.b200_internal_set_gemm_skinny(ctx.h, 1)
    assert rel(out32, tile) < 1e-5


def _few_row_hook(ctx):
    f = ctx.lib.b200_internal_few_row_gemm
    vp, i, z, fl = bridge._vp, bridge._i, bridge.C.c_size_t, bridge.C.c_float
    f.argtypes = [vp, vp, vp, vp, z, z, z, vp, vp, vp, vp, vp, i, fl, i, vp, vp, i, i, i]
    f.restype = i
    return f


def _produce(ctx, A, W, res, wn, M, N, K):
    """Producer half on the GPU: h = res + A W, xw = h * wn, row sums (2^-32 fixed point, 64-bit; two fp32 words each here)."""
    f = _few_row_hook(ctx)
    h, xw = ctx.empty((M, N), "bf16"), ctx.empty((M, N), "bf16")
    stats = ctx.array(np.zeros((M, 2, 2), np.float32))
    ctx._check(f(ctx.h, ctx.array(A, "bf16").ptr, ctx.array(W, "bf16").ptr, h.ptr, M, N, K, ctx.array(res, "bf16").ptr,
                 ctx.array(wn, "bf16").ptr, xw.ptr, stats.ptr, None, 0, 0.0, 0, None, None, 0, 0, 0))
    return h, xw, stats


def _sums(stats):
    return stats.download().view(np.uint64).reshape(-1, 2).astype(np.float64) / 2.0 ** 32


@pytest.mark.parametrize("M", [1, 5, 32, 64])
@pytest.mark.parametrize("N,K,N2,double", [(2048, 2048, 3072, 1), (2048, 5632, 32000, 0), (128, 256, 104, 1), (72, 64, 72, 0), (2048, 2048, 2048, 0)])
def test_few_row_kernel_residual_and_split_normalisation(ctx, M, N, K, N2, double):
    """Decode epilogues of the few-row kernel.  Producer: h = residual + A W, h * w_norm and the rows' sums of squares per
    row.  Consumer: rstd * ((h * w_norm) W2), with the attention's second unit norm when `double` (RMSNorm forward of
    cpp/src/RMSNorm.cpp applied twice) -- against numpy in float64 with the same bf16 roundings of the stored tensors."""
    eps = 1e-5
    A, W = _ab(M, N, K, False, False, std_b=0.05)
    res = synth.bf16_round(synth.normal(SEED, f"res{M}{N}", (M, N)) * (1.0 + np.arange(M, dtype=np.float32)[:, None] / 7.0))
    wn = synth.bf16_round(1.0 + 0.2 * synth.normal(SEED, f"wn{N}", (N,)))
    W2 = synth.bf16_round(synth.normal(SEED, f"W2{N}{N2}", (N, N2), 0.05))
    h_dev, xw_dev, stats_dev = _produce(ctx, A, W, res, wn, M, N, K)
    h, xw, stats = h_dev.download(), xw_dev.download(), _sums(stats_dev)
    exp_h = _ref(A, W, False, False) + res
    assert rel(h, exp_h) < 4e-3
    np.testing.assert_array_equal(xw, synth.bf16_round(h * wn))                       # from the values as stored
    hs = h.astype(np.float64)
    np.testing.assert_allclose(stats[:, 0], (hs * hs).sum(-1), rtol=1e-5)
    np.testing.assert_allclose(stats[:, 1], (xw.astype(np.float64) ** 2).sum(-1), rtol=1e-5)
    # consumer
    y = xw.astype(np.float64) / np.sqrt((hs * hs).mean(-1, keepdims=True) + eps)
    if double:
        y = y / np.sqrt((y * y).mean(-1, keepdims=True) + eps)
    exp = y @ W2.astype(np.float64)
    out = ctx.empty((M, N2), "bf16")
    ctx._check(_few_row_hook(ctx)(ctx.h, xw_dev.ptr, ctx.array(W2, "bf16").ptr, out.ptr, M, N2, N, None, None, None, None,
                                  stats_dev.ptr, double, eps, 0, None, None, 0, 0, 0))
    got = out.download()
    assert rel(got, exp) < 5e-3, rel(got, exp)
    assert np.abs(got - exp).max() < 2e-2 * np.abs(exp).max()


@pytest.mark.parametrize("M,I,H", [(3, 5632, 2048), (32, 5632, 2048), (64, 704, 256), (17, 64, 128)])
def test_few_row_kernel_swiglu_on_a_normalised_row(ctx, M, I, H):
    eps = 1e-5
    A, W = _ab(M, H, 192, False, False, std_b=0.3)
    res = synth.bf16_round(synth.normal(SEED, f"sres{M}{H}", (M, H), 2.0))
    wn = synth.bf16_round(1.0 + 0.2 * synth.normal(SEED, f"swn{H}", (H,)))
    Wgu = synth.bf16_round(synth.normal(SEED, f"sW{H}{I}", (H, 2 * I), 0.03))
    h_dev, xw_dev, stats_dev = _produce(ctx, A, W, res, wn, M, H, 192)
    hs, xw = h_dev.download().astype(np.float64), xw_dev.download().astype(np.float64)
    gu = (xw / np.sqrt((hs * hs).mean(-1, keepdims=True) + eps)) @ Wgu.astype(np.float64)
    g, u = gu[:, :I], gu[:, I:]
    exp = g / (1.0 + np.exp(-g)) * u
    out = ctx.empty((M, I), "bf16")
    ctx._check(_few_row_hook(ctx)(ctx.h, xw_dev.ptr, ctx.array(Wgu, "bf16").ptr, out.ptr, M, 2 * I, H, None, None, None, None,
                                  stats_dev.ptr, 0, eps, I, None, None, 0, 0, 0))
    assert rel(out.download(), exp) < 8e-3


@pytest.mark.parametrize("M,hd,pos", [(4, 128, 37), (32, 64, 5), (7, 6, 3)])
def test_few_row_kernel_rotary_epilogue_on_a_normalised_row(ctx, M, hd, pos):
    """Q and K columns rotated at one position (RoPE::forward, cpp/src/Positional.cpp: interleaved pairs), V columns left alone."""
    eps, H = 1e-5, 256
    nq, nkv = 4, 2
    N, cols = (nq + 2 * nkv) * hd, (nq + nkv) * hd
    A, W = _ab(M, H, 128, False, False, std_b=0.3)
    res = synth.bf16_round(synth.normal(SEED, f"rres{M}", (M, H)))
    wn = synth.bf16_round(1.0 + 0.2 * synth.normal(SEED, "rwn", (H,)))
    Wqkv = synth.bf16_round(synth.normal(SEED, f"rW{N}", (H, N), 0.05))
    h_dev, xw_dev, stats_dev = _produce(ctx, A, W, res, wn, M, H, 128)
    hs, xw = h_dev.download().astype(np.float64), xw_dev.download().astype(np.float64)
    half = hd // 2
    ang = np.arange(64)[:, None] * (10000.0 ** (-np.arange(half) / half))[None, :]
    cos_t, sin_t = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    y = xw / np.sqrt((hs * hs).mean(-1, keepdims=True) + eps)
    y = (y / np.sqrt((y * y).mean(-1, keepdims=True) + eps)) @ Wqkv.astype(np.float64)
    exp = y.copy()
    r = y[:, :cols].reshape(M, -1, half, 2)
    c, s_ = cos_t[pos].astype(np.float64), sin_t[pos].astype(np.float64)
    exp[:, :cols] = np.stack([r[..., 0] * c - r[..., 1] * s_, r[..., 0] * s_ + r[..., 1] * c], -1).reshape(M, cols)
    out = ctx.empty((M, N), "bf16")
    ctx._check(_few_row_hook(ctx)(ctx.h, xw_dev.ptr, ctx.array(Wqkv, "bf16").ptr, out.ptr, M, N, H, None, None, None, None,
                                  stats_dev.ptr, 1, eps, 0, ctx.array(cos_t).ptr, ctx.array(sin_t).ptr, hd, cols, pos))
    assert rel(out.download(), exp) < 6e-3


PROJ = [("qkv", 2048, 3072), ("o", 2048, 2048), ("gate_up", 2048, 11264), ("down", 5632, 2048)]


@pytest.mark.parametrize("name,K,N", PROJ)
def test_full_size_projection_shapes(ctx, name, K, N):
    """M = 16384 tokens, the three GEMM forms of one projection, checked on sampled rows/cols."""
    M = 16384
    rng = np.random.default_rng(1)
    x = ctx.empty((M, K), "bf16"); w = ctx.empty((K, N), "bf16"); dy = ctx.empty((M, N), "bf16")
    lib = ctx.lib
    ctx._check(lib.b200_fill_normal(ctx.h, x.ptr, 1, M * K, 11, 1.0))
    ctx._check(lib.b200_fill_normal(ctx.h, w.ptr, 1, K * N, 12, 0.02))
    ctx._check(lib.b200_fill_normal(ctx.h, dy.ptr, 1, M * N, 13, 1.0))
    hx, hw, hdy = x.download(), w.download(), dy.download()
    def worst(got, exp):     # largest element error against the largest reference element (a wrong tile cannot hide in an L2 ratio)
        return float(np.abs(got.astype(np.float64) - exp).max() / np.abs(exp).max())

    y = ctx.gemm(x, w, M, N, K, out_dtype="bf16").download()                     # forward  NN
    # rows from every 256-row tile pair boundary region and at random
    rows = np.unique(np.concatenate([rng.choice(M, 24, replace=False), [0, 127, 128, 255, 256, M - 129, M - 1]]))
    exp = hx[rows].astype(np.float64) @ hw.astype(np.float64)
    assert rel(y[rows], exp) < 5e-3 and worst(y[rows], exp) < 8e-3
    dx = ctx.gemm(dy, w, M, K, N, False, True, out_dtype="bf16").download()      # dgrad    NT
    exp = hdy[rows].astype(np.float64) @ hw.astype(np.float64).T
    assert rel(dx[rows], exp) < 5e-3 and worst(dx[rows], exp) < 8e-3
    dw = ctx.gemm(x, dy, K, N, M, True, False, out_dtype="f32").download()       # wgrad    TN
    cols = np.unique(np.concatenate([rng.choice(N, 16, replace=False), [0, 255, 256, N - 1]]))
    exp = hx.astype(np.float64).T @ hdy[:, cols].astype(np.float64)
    assert rel(dw[:, cols], exp) < 1e-4 and worst(dw[:, cols], exp) < 1e-3
    # every output element is finite and no 256x256 tile was left unwritten (a skipped tile would keep the fill value)
    assert np.isfinite(y).all() and np.isfinite(dx).all() and np.isfinite(dw).all()


@pytest.mark.parametrize("M,I,K,want", [(4096, 1024, 512, True), (4096, 1024, 512, False), (2560, 2080, 200, True),
                                         (32, 1024, 512, False), (7, 96, 64, False), (32, 1024, 512, True), (300, 96, 64, True)])
def test_ffn_gemm_with_the_activation_in_the_epilogue(ctx, M, I, K, want):
    """silu(x Wg) * (x Wu) on W = [gate | up]: two-CTA kernel (large M), few-row kernel (M <= 64, products not
    wanted) and the GEMM + SwiGLU pair must agree; gate/up products equal the plain GEMM's bit for bit."""
    x = synth.bf16_round(synth.normal(SEED, f"ffnx{M}{K}", (M, K)))
    w = synth.bf16_round(synth.normal(SEED, f"ffnw{K}{I}", (K, 2 * I), 0.05))
    dx, dw = ctx.array(x, "bf16"), ctx.array(w, "bf16")
    res = ctx.gemm_ffn(dx, dw, M, I, K, want_gate_up=want)
    act = (res[0] if want else res).download()
    plain = ctx.gemm(dx, dw, M, 2 * I, K, out_dtype="bf16").download()
    g, u = plain[:, :I].astype(np.float32), plain[:, I:].astype(np.float32)
    ref_act = synth.bf16_round(g / (1.0 + np.exp(-g)) * u)
    if want:
        np.testing.assert_array_equal(res[1].download(), plain)
        assert rel(act, ref_act) < 6e-3                     # the epilogue activates the fp32 accumulators, the reference the rounded products
        exact = x.astype(np.float64) @ w.astype(np.float64)
        assert rel(act, exact[:, :I] / (1.0 + np.exp(-exact[:, :I])) * exact[:, I:]) < 5e-3
    else:
        exact = x.astype(np.float64) @ w.astype(np.float64)
        ge, ue = exact[:, :I], exact[:, I:]
        assert rel(act, ge / (1.0 + np.exp(-ge)) * ue) < 8e-3
