"""Autoregressive decode with a KV cache and the sampler.
* greedy token ids of the fp32 engine are bit-exact against the CPU checker, which (like the reference's
  Python generate loop, python/pipeline/inference/sampler.py:115-148) re-runs the full context per token;
* the bf16 cache path reproduces the engine's own full-context forward (logits within 2e-2, same greedy ids);
* the sampler's deterministic filters (repetition penalty, top-k, top-p) match a numpy restatement of
  sampler.py:43-98 exactly (threshold and kept count; the restatement itself is pinned in test_sampler_golden.py);
  the random draw is pinned only by seed self-consistency and by staying inside the kept set (the reference draws
  with MLX's RNG: unpinned)."""
import numpy as np
import pytest

from gpu_util import BF16_TOL, bridge, ctx, rel, synth  # noqa: F401
from oracle import oracle
from sampler_rules import ref_filters

pytestmark = pytest.mark.gpu


# 32000: the benchmark model; 100352: the vocabulary of the reference's own training configurations
# (cpp/src/RunTrainer.cpp:121), which does not fit in shared memory
@pytest.mark.parametrize("V", [32000, 100352])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("top_k,top_p,penalty", [(0, 1.0, 1.0), (50, 1.0, 1.0), (0, 0.9, 1.0), (50, 0.9, 1.1), (0, 0.9, 1.1), (1, 0.5, 1.3)])
def test_sampler_filters_match_the_reference_rules(ctx, dtype, top_k, top_p, penalty, V):
    B, Lh = 6, 200
    lg = synth.normal(4, "logits", (B, V), 2.5)
    lg[1] *= 4.0                      # one peaked row
    lg[2] = np.round(lg[2])           # many exact ties
    if dtype == "bf16":
        lg = synth.bf16_round(lg)
    hist = synth.token_ids(4, "hist", (B, Lh + 8), V)
    hist[:, -140:-130] = 220          # whitespace ids inside and outside the window
    ws = (220, 256, 198, 385)
    cfg = bridge.SamplerConfig.make(temperature=0.0, top_p=top_p, repetition_penalty=penalty, top_k=top_k, whitespace_ids=ws)
    tok, thr, kept = ctx.sample(ctx.array(lg, dtype), ctx.array(hist, "i32"), Lh, cfg)
    tok, thr, kept = tok.download(), thr.download(), kept.download()
    for b in range(B):
        pen, filt = ref_filters(lg[b], hist[b, :Lh], penalty, top_k, top_p, ws)
        exp_kept = int(np.isfinite(filt).sum())
        # the cumulative-probability crossing can move by one rank under a different summation order
        assert abs(int(kept[b]) - exp_kept) <= max(1, exp_kept // 500), (b, kept[b], exp_kept)
        if int(kept[b]) == exp_kept:
            assert thr[b] == (filt[np.isfinite(filt)].min() if exp_kept < V else thr[b])
        assert tok[b] == int(np.argmax(pen)), "greedy = lowest id among the maxima of the penalised logits"


@pytest.mark.parametrize("top_k,top_p,penalty", [(0, 0.9, 1.1), (50, 0.9, 1.0)])
def test_sampler_filters_beyond_two_to_the_seventeenth_entries(ctx, top_k, top_p, penalty):
    """From 131072 vocabulary entries on, a histogram bin's probability mass is kept in one 64-bit counter instead of
    three 32-bit pieces (which could overflow); same rules, same checker."""
    B, Lh, V = 3, 150, 140000
    lg = synth.normal(14, "logits_wide", (B, V), 2.5)
    lg[1] *= 3.0
    hist = synth.token_ids(14, "hist_wide", (B, Lh + 8), V)
    ws = (220, 256, 198, 385)
    cfg = bridge.SamplerConfig.make(temperature=0.0, top_p=top_p, repetition_penalty=penalty, top_k=top_k, whitespace_ids=ws)
    tok, thr, kept = ctx.sample(ctx.array(lg, "f32"), ctx.array(hist, "i32"), Lh, cfg)
    tok, thr, kept = tok.download(), thr.download(), kept.download()
    for b in range(B):
        pen, filt = ref_filters(lg[b], hist[b, :Lh], penalty, top_k, top_p, ws)
        exp_kept = int(np.isfinite(filt).sum())
        assert abs(int(kept[b]) - exp_kept) <= max(1, exp_kept // 500), (b, kept[b], exp_kept)
        if int(kept[b]) == exp_kept and exp_kept < V:
            assert abs(thr[b] - filt[np.isfinite(filt)].min()) <= 1e-6 * max(1.0, abs(thr[b]))
        assert tok[b] == int(np.argmax(pen))


def test_sampling_draw_is_seeded_and_stays_in_the_nucleus(ctx):
    B, V = 32, 4096
    base = synth.normal(8, "lg", (1, V), 2.0)
    lg = np.repeat(base, B, 0)
    cfg = bridge.SamplerConfig.make(temperature=0.8, top_p=0.9, repetition_penalty=1.0, top_k=0, seed=1234)
    d = ctx.array(lg, "f32")
    t1 = ctx.sample(d, None, 0, cfg, step=7)[0].download()
    t2 = ctx.sample(d, None, 0, cfg, step=7)[0].download()
    t3 = ctx.sample(d, None, 0, cfg, step=8)[0].download()
    np.testing.assert_array_equal(t1, t2)                      # same (seed, step, row) -> same token
    assert (t1 != t3).any()
    _, filt = ref_filters(lg[0], [], 1.0, 0, 0.9)
    assert np.isfinite(filt[t1]).all() and np.isfinite(filt[t3]).all()
    assert len(set(t1.tolist())) > 4                           # rows draw independently
    # the empirical distribution over many (row, step) draws follows softmax(logits / T) on the nucleus
    draws = np.concatenate([ctx.sample(d, None, 0, cfg, step=s)[0].download() for s in range(64)])
    w = np.where(np.isfinite(filt), np.exp((lg[0] - lg[0].max()) / 0.8), 0.0)
    p = w / w.sum()
    top = np.argsort(-p)[:5]
    freq = np.array([(draws == t).mean() for t in top])
    assert np.abs(freq - p[top]).max() < 0.03


def test_fp32_greedy_decode_is_bit_exact_against_the_checker(ctx, orc):
    B, P, NEW = 3, 7, 6
    shape = dict(H=128, I=96, nH=4, nKV=2, hd=32, V=97, L=2)
    params = synth.model_params(21, oracle.Config(B=B, S=P + NEW, **shape), std=0.3)
    prompt = synth.token_ids(21, "prompt", (B, P), shape["V"])
    model = bridge.Model(ctx, bridge.Shape(B=B, S=P + NEW, **shape), "f32", with_optimizer=False)
    model.load_params(params)
    got, _, _ = model.generate(prompt, NEW, bridge.SamplerConfig.make(temperature=0.0))
    ctxt = prompt.copy()
    for t in range(NEW):
        cfg = oracle.Config(B=B, S=ctxt.shape[1], **shape)
        _, _, logits = orc.model_loss_and_grads(cfg, ctxt, np.zeros_like(ctxt), params, want_grads=False, want_logits=True)
        nxt = logits.reshape(B, ctxt.shape[1], -1)[:, -1].argmax(-1).astype(np.int32)
        np.testing.assert_array_equal(got[:, t], nxt, err_msg=f"generated token {t}")
        ctxt = np.concatenate([ctxt, nxt[:, None]], 1)
    model.close()


def test_generate_again_with_a_longer_total_length_and_a_larger_batch(ctx):
    """The K/V caches grow when a later call asks for more than the first one allocated."""
    shape = dict(H=128, I=96, nH=4, nKV=2, hd=32, V=211, L=2)
    model = bridge.Model(ctx, bridge.Shape(B=4, S=64, **shape), "f32", with_optimizer=False)
    model.init_synthetic(3, 0.3)
    greedy = bridge.SamplerConfig.make(temperature=0.0)
    p_small = synth.token_ids(31, "p", (2, 6), shape["V"])
    first, _, _ = model.generate(p_small, 4, greedy)
    p_big = np.concatenate([p_small, synth.token_ids(32, "p2", (2, 6), shape["V"])], 0)
    longer, _, _ = model.generate(p_big, 20, greedy)              # batch 2 -> 4, total length 10 -> 26
    np.testing.assert_array_equal(longer[:2, :4], first)           # same prompts decode to the same ids
    again, _, _ = model.generate(p_small, 4, greedy)
    np.testing.assert_array_equal(again, first)
    model.close()


def test_generate_with_a_vocabulary_larger_than_shared_memory(ctx, orc):
    """The reference's own configurations use 100256 / 100352 ids: greedy ids bit-exact against the checker in fp32,
    and the captured bf16 decode step with sampling is reproducible and stays inside the vocabulary."""
    B, P, NEW, V = 2, 5, 4, 100352
    shape = dict(H=64, I=96, nH=2, nKV=1, hd=32, V=V, L=1)
    params = synth.model_params(23, oracle.Config(B=B, S=P + NEW, **shape), std=0.3)
    prompt = synth.token_ids(23, "prompt", (B, P), V)
    model = bridge.Model(ctx, bridge.Shape(B=B, S=P + NEW, **shape), "f32", with_optimizer=False)
    model.load_params(params)
    got, _, _ = model.generate(prompt, NEW, bridge.SamplerConfig.make(temperature=0.0))
    ctxt = prompt.copy()
    for t in range(NEW):
        cfg = oracle.Config(B=B, S=ctxt.shape[1], **shape)
        _, _, logits = orc.model_loss_and_grads(cfg, ctxt, np.zeros_like(ctxt), params, want_grads=False, want_logits=True)
        nxt = logits.reshape(B, ctxt.shape[1], -1)[:, -1].argmax(-1).astype(np.int32)
        np.testing.assert_array_equal(got[:, t], nxt, err_msg=f"generated token {t}")
        ctxt = np.concatenate([ctxt, nxt[:, None]], 1)
    model.close()
    model = bridge.Model(ctx, bridge.Shape(B=B, S=P + 8, **shape), "bf16", with_optimizer=False)
    model.init_synthetic(5, 0.05)
    cfg = bridge.SamplerConfig.make(temperature=0.8, top_p=0.9, repetition_penalty=1.1, seed=9, whitespace_ids=(220, 256, 198, 385))
    a, _, _ = model.generate(prompt, 8, cfg)
    b, _, _ = model.generate(prompt, 8, cfg)
    np.testing.assert_array_equal(a, b)
    assert a.min() >= 0 and a.max() < V
    model.close()


@pytest.mark.parametrize("hd,nH,nKV", [(128, 4, 2), (64, 4, 1), (64, 6, 2), (32, 8, 8)])   # groups of 2, 4, 3 (separate cache append), 1
def test_bf16_cache_decode_matches_full_context_forward(ctx, hd, nH, nKV):
    B, P, NEW = 4, 40, 6
    shape = dict(H=nH * hd, I=768, nH=nH, nKV=nKV, hd=hd, V=1024, L=2)
    S = P + NEW
    model = bridge.Model(ctx, bridge.Shape(B=B, S=S, **shape), "bf16", with_optimizer=False)
    model.init_synthetic(5, 0.05)
    prompt = synth.token_ids(5, "prompt", (B, P), shape["V"])
    model.decode_begin(B, S)
    logits = model.prefill(ctx.array(prompt, "i32"), B, P).download()
    ctxt = prompt.copy()
    for t in range(NEW):
        full = model.forward(ctx.array(ctxt, "i32"), B, ctxt.shape[1]).download().reshape(B, ctxt.shape[1], -1)[:, -1]
        assert rel(logits, full) < BF16_TOL, (t, rel(logits, full))
        nxt = full.argmax(-1).astype(np.int32)
        gap = np.sort(full, -1)[:, -1] - np.sort(full, -1)[:, -2]
        clear = gap > 0.05 * np.abs(full).max()
        np.testing.assert_array_equal(logits.argmax(-1)[clear], nxt[clear])
        logits = model.decode_step(ctx.array(nxt, "i32"), B, P + t).download()
        ctxt = np.concatenate([ctxt, nxt[:, None]], 1)
    model.close()

@pytest.mark.parametrize("B", [3, 40, 64])          # 32- and 64-row forms of the few-row projections
def test_decode_step_with_norms_inside_the_projections_matches_the_separate_kernels(ctx, B, monkeypatch):
    """By default the residual adds and RMS norms of a decode step ride in the few-row projections (the producer of the
    residual stream leaves h * w_norm and the rows' sums of squares, the consumer scales by rstd).  The logits must agree
    with the step that runs them as kernels of their own, and with the full-context forward, and take fewer launches."""
    P, NEW = 24, 4
    shape = dict(H=256, I=512, nH=4, nKV=2, hd=64, V=1024, L=3)
    S = P + NEW
    model = bridge.Model(ctx, bridge.Shape(B=B, S=S, **shape), "bf16", with_optimizer=False)
    model.init_synthetic(11, 0.05)
    prompt = synth.token_ids(11, "prompt", (B, P), shape["V"])

    def run(folded, forced=None):
        monkeypatch.setenv("B200_DECODE_FOLD_NORM", "1" if folded else "0")
        model.decode_begin(B, S)
        logits = model.prefill(ctx.array(prompt, "i32"), B, P).download()
        out, ids = [], []
        n0 = ctx.launch_count()
        for t in range(NEW):
            nxt = logits.argmax(-1).astype(np.int32) if forced is None else forced[t]
            ids.append(nxt)
            logits = model.decode_step(ctx.array(nxt, "i32"), B, P + t).download()
            out.append(logits)
        return out, ids, ctx.launch_count() - n0

    try:
        fold_out, ids, n_fold = run(True)
        sep_out, _, n_sep = run(False, ids)
        for t, (a, b) in enumerate(zip(fold_out, sep_out)):
            assert rel(a, b) < 1e-2, (t, rel(a, b))
        ctxt = np.concatenate([prompt] + [i[:, None] for i in ids], 1)
        full = model.forward(ctx.array(ctxt, "i32"), B, ctxt.shape[1]).download().reshape(B, ctxt.shape[1], -1)[:, -1]
        assert rel(fold_out[-1], full) < BF16_TOL
        assert n_fold == n_sep - NEW * 2 * shape["L"]           # two norm kernels fewer per layer and step
    finally:
        model.close()


@pytest.mark.parametrize("nH,nKV,P", [(4, 2, 150), (8, 2, 700), (8, 1, 130), (4, 2, 1100)])   # groups of 2, 4, 8, 2; 2, 6, 2 and 9 cache tiles
def test_tensor_core_decode_attention(ctx, nH, nKV, P, monkeypatch):
    """With enough (sequence, KV head) pairs to fill the GPU, head_dim 128 decode attention runs on the tensor cores
    (whole-tile TMA reads of the cache, ring reuse beyond five tiles, a ragged last tile, a cache length that is not
    a multiple of the tile).  Checked against the engine's full-context forward, against the CUDA-core kernel, and
    captured (position on the device) against eagerly enqueued."""
    hd, NEW = 128, 5
    import torch
    B = torch.cuda.get_device_properties(0).multi_processor_count // (2 * nKV) + 1      # just enough pairs to qualify
    shape = dict(H=nH * hd, I=512, nH=nH, nKV=nKV, hd=hd, V=512, L=2)
    S = P + NEW
    model = bridge.Model(ctx, bridge.Shape(B=B, S=S, **shape), "bf16", with_optimizer=False)
    model.init_synthetic(6, 0.05)
    prompt = synth.token_ids(6, "prompt", (B, P), shape["V"])
    ctx.lib.b200_internal_set_attn_decode_tc.argtypes = [bridge._vp, bridge._i]

    def run(tc):
        ctx.lib.b200_internal_set_attn_decode_tc(ctx.h, tc)
        model.decode_begin(B, S)
        logits = model.prefill(ctx.array(prompt, "i32"), B, P).download()
        out, ctxt = [], prompt.copy()
        for t in range(NEW):
            nxt = logits.argmax(-1).astype(np.int32) if tc else forced[t]
            out.append((logits, nxt))
            logits = model.decode_step(ctx.array(nxt, "i32"), B, P + t).download()
            ctxt = np.concatenate([ctxt, nxt[:, None]], 1)
        out.append((logits, None))
        return out, ctxt

    try:
        n0 = ctx.launch_count()
        tc_out, ctxt = run(1)
        forced = [nxt for _, nxt in tc_out[:-1]]
        core_out, _ = run(0)
        for t, ((a, _), (b, _)) in enumerate(zip(tc_out, core_out)):
            assert rel(a, b) < BF16_TOL, (t, rel(a, b))       # two bf16 kernels: P rounded to bf16 here, fp32 there
        full = model.forward(ctx.array(ctxt, "i32"), B, ctxt.shape[1]).download().reshape(B, ctxt.shape[1], -1)[:, -1]
        assert rel(tc_out[-1][0], full) < BF16_TOL
        ctx.lib.b200_internal_set_attn_decode_tc(ctx.h, 1)
        cfg = bridge.SamplerConfig.make(temperature=0.0, top_p=1.0, repetition_penalty=1.0, top_k=0)
        graph_ids, _, _ = model.generate(prompt, NEW, cfg)
        monkeypatch.setenv("B200_DECODE_GRAPH", "0")
        eager_ids, _, _ = model.generate(prompt, NEW, cfg)
        np.testing.assert_array_equal(graph_ids, eager_ids)
    finally:
        ctx.lib.b200_internal_set_attn_decode_tc(ctx.h, 1)
        model.close()


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_captured_decode_step_equals_the_eagerly_enqueued_one(ctx, temperature, monkeypatch):
    """generate() replays one captured step (position read on the device); the ids must equal those of the
    step-by-step enqueued loop, for greedy and for seeded sampling."""
    B, P, NEW = 5, 37, 14
    shape = dict(H=256, I=512, nH=4, nKV=2, hd=64, V=2048, L=3)
    model = bridge.Model(ctx, bridge.Shape(B=B, S=P + NEW, **shape), "bf16", with_optimizer=False)
    model.init_synthetic(9, 0.08)
    prompt = synth.token_ids(9, "prompt", (B, P), shape["V"])
    cfg = bridge.SamplerConfig.make(temperature=temperature, top_p=0.9, repetition_penalty=1.1, top_k=40, seed=77, whitespace_ids=(3, 4))
    n0 = ctx.launch_count()
    graph_ids, _, _ = model.generate(prompt, NEW, cfg)
    n_graph = ctx.launch_count() - n0
    monkeypatch.setenv("B200_DECODE_GRAPH", "0")
    n0 = ctx.launch_count()
    eager_ids, _, _ = model.generate(prompt, NEW, cfg)
    n_eager = ctx.launch_count() - n0
    np.testing.assert_array_equal(graph_ids, eager_ids)
    assert graph_ids.min() >= 0 and graph_ids.max() < shape["V"]
    assert n_graph == n_eager + (NEW - 1)          # same kernels, plus the position increment of each captured-mode step
    model.close()
