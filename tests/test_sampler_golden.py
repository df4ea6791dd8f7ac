"""The sampler's deterministic rules against outputs of the reference's own sampler functions
(tests/golden/sampler_reference_rules.npz, written by tests/golden/make_sampler_golden.py from
python/pipeline/inference/sampler.py running on a numpy stand-in for mlx.core):
* the numpy restatement the GPU tests use as their checker reproduces them exactly (no GPU needed);
* the on-device sampler reproduces them: greedy id, kept count, threshold."""
import os

import numpy as np
import pytest

from sampler_rules import ref_filters

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampler_reference_rules.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def cases(g):
    ws = tuple(int(w) for w in g["whitespace_ids"])
    for r in range(int(g["n_rows"])):
        lg, hist, res = g[f"logits.{r}"], g[f"history.{r}"], g[f"results.{r}"]
        for c, (top_k, top_p, penalty) in enumerate(g["configs"]):
            yield r, c, lg, hist, int(top_k), float(top_p), float(penalty), ws, res[c], g[f"pen_ids.{r}.{c}"], g[f"pen_vals.{r}.{c}"]


def test_numpy_restatement_reproduces_the_reference_sampler(golden):
    n = 0
    for r, c, lg, hist, top_k, top_p, penalty, ws, (thr, kept, greedy), pen_ids, pen_vals in cases(golden):
        pen, filt = ref_filters(lg, hist, penalty, min(top_k, lg.size), top_p, ws)
        changed = np.nonzero(pen != lg)[0]
        np.testing.assert_array_equal(changed, pen_ids, err_msg=f"row {r} config {c}: penalised ids")
        np.testing.assert_array_equal(pen[changed], pen_vals, err_msg=f"row {r} config {c}: penalised values")
        keep = np.isfinite(filt)
        assert int(keep.sum()) == int(kept), (r, c)
        if kept < lg.size:
            assert float(filt[keep].min()) == thr, (r, c)
        assert int(np.argmax(pen)) == int(greedy), (r, c)
        n += 1
    assert n == 70


@pytest.mark.gpu
def test_device_sampler_reproduces_the_reference_sampler(golden):
    from gpu_util import bridge
    ctx = bridge.Context(0)
    try:
        for r, c, lg, hist, top_k, top_p, penalty, ws, (thr, kept, greedy), _, _ in cases(golden):
            V = lg.size
            cfg = bridge.SamplerConfig.make(temperature=0.0, top_p=top_p, repetition_penalty=penalty, top_k=min(top_k, V), whitespace_ids=ws)
            h = np.concatenate([hist, np.zeros(8, np.int32)])[None, :]
            tok, dthr, dkept = ctx.sample(ctx.array(lg[None, :], "f32"), ctx.array(h, "i32"), hist.size, cfg)
            tok, dthr, dkept = int(tok.download()[0]), float(dthr.download()[0]), int(dkept.download()[0])
            assert tok == int(greedy), (r, c, tok, greedy)
            # a cumulative sum taken in another order can move the top-p crossing by one rank
            assert abs(dkept - int(kept)) <= max(1, int(kept) // 500), (r, c, dkept, kept)
            if dkept == int(kept) and kept < V:
                assert abs(dthr - thr) <= 1e-6 * max(1.0, abs(thr)), (r, c, dthr, thr)
    finally:
        ctx.close()
