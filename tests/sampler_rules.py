"""numpy restatement of the deterministic part of the reference's sampler
(python/pipeline/inference/sampler.py:43-98): repetition penalty over the last 128 ids (whitespace ids exempt),
top-k, top-p.  Test infrastructure: pinned against outputs of the reference's own functions in
tests/test_sampler_golden.py and used as the checker of the on-device sampler."""
import numpy as np


def ref_filters(logits, generated, penalty, top_k, top_p, whitespace=(), window=128):
    """Returns (penalised logits, filtered logits with -inf outside the kept set), float32."""
    lg = np.asarray(logits, np.float32).copy()
    if penalty != 1.0 and len(generated):
        seen = set(int(t) for t in generated[-window:]) - set(whitespace)
        for t in seen:
            v = float(lg[t])              # the reference edits a Python list of floats (double) and converts back (sampler.py:62-69)
            lg[t] = np.float32((v / penalty if v > 0.0 else v * penalty) - (penalty - 1.0) * 35.0)
    pen = lg.copy()
    if top_k > 0:
        thr = np.sort(lg)[-top_k]
        lg = np.where(lg >= thr, lg, -np.inf).astype(np.float32)
    if top_p < 1.0:
        order = np.argsort(-lg, kind="stable")
        s = lg[order]
        p = np.exp(s - s[0], dtype=np.float32)
        p = p / p.sum(dtype=np.float32)
        cum = np.cumsum(p, dtype=np.float32)
        idx = np.nonzero(cum > np.float32(top_p))[0]     # the comparison is made on Python floats of the float32 values (sampler.py:90-92)
        if len(idx):
            cutoff = max(1, int(idx[0]))
            lg = np.where(lg >= s[cutoff], lg, -np.inf).astype(np.float32)
    return pen, lg
