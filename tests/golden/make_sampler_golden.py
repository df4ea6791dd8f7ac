"""Generates tests/golden/sampler_reference_rules.npz: the reference's OWN sampler functions
(python/pipeline/inference/sampler.py: apply_repetition_penalty, apply_top_k, apply_top_p and sample_token at
temperature 0) run on seeded logits.

MLX cannot be installed where this runs, so `mlx.core` is replaced by the small numpy stand-in below before the
reference module is imported: float32 arrays whose sort / argsort / softmax / cumsum / where / argmax are numpy's.
The control flow, the rules and their order are the reference's unmodified code; only the array arithmetic under them
is numpy's float32 (a cumulative sum in another order can move the top-p crossing by one rank; the tests allow that).
The random draw (mx.random.categorical) is not reproduced: no fixture depends on it.

Usage:  REFERENCE_ROOT=<checkout of the reference> python tests/golden/make_sampler_golden.py"""
import importlib.util
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


class array:                                   # the part of mx.array the sampler touches
    def __init__(self, v, dtype=None):
        v = v.v if isinstance(v, array) else v
        a = np.asarray(v)
        if dtype is not None:
            a = a.astype(dtype)
        elif a.dtype.kind == "f":
            a = a.astype(np.float32)
        self.v = a

    def tolist(self): return self.v.tolist()
    def item(self): return self.v.item()
    def __neg__(self): return array(-self.v)
    def __ge__(self, o): return array(self.v >= _raw(o))
    def __truediv__(self, o): return array((self.v / np.float32(_raw(o))).astype(np.float32))
    def __getitem__(self, i): return array(self.v[_raw(i)])
    def __len__(self): return len(self.v)


def _raw(x): return x.v if isinstance(x, array) else x


def _softmax(a, axis=-1):
    x = _raw(a).astype(np.float32)
    e = np.exp(x - x.max(), dtype=np.float32)
    return array(e / e.sum(dtype=np.float32))


mx = types.ModuleType("mlx.core")
mx.array = array
mx.int32, mx.float32 = np.int32, np.float32
mx.sort = lambda a: array(np.sort(_raw(a)))
mx.argsort = lambda a: array(np.argsort(_raw(a), kind="stable"))
mx.where = lambda c, a, b: array(np.where(_raw(c), _raw(a), _raw(b)).astype(np.float32))
mx.softmax = _softmax
mx.cumsum = lambda a: array(np.cumsum(_raw(a), dtype=np.float32))
mx.argmax = lambda a, axis=-1: array(np.argmax(_raw(a), axis=axis))
mx.eval = lambda *a: None
mlx = types.ModuleType("mlx")
mlx.core = mx
sys.modules["mlx"], sys.modules["mlx.core"] = mlx, mx


def load_reference_sampler():
    root = os.environ.get("REFERENCE_ROOT") or os.path.join(HERE, "..", "..", "..", "reference")
    path = os.path.join(root, "python", "pipeline", "inference", "sampler.py")
    if not os.path.exists(path):
        raise SystemExit(f"reference sampler not found at {path}: set REFERENCE_ROOT")
    spec = importlib.util.spec_from_file_location("reference_sampler", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["reference_sampler"] = mod          # dataclasses looks the module up while the class body runs
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = load_reference_sampler()
    rng = np.random.default_rng(20250)
    ws = [220, 256, 198, 385]
    out = {"whitespace_ids": np.asarray(ws, np.int32)}
    configs = ((0, 1.0, 1.0), (50, 1.0, 1.0), (0, 0.9, 1.0), (50, 0.9, 1.15), (0, 0.9, 1.1), (1, 0.5, 1.3), (5, 0.3, 1.0))
    out["configs"] = np.asarray(configs, np.float64)               # rows of (top_k, top_p, repetition_penalty)
    rows = []
    for V, kinds in ((64, ("normal", "peaked", "ties")), (1000, ("normal", "peaked", "ties")), (4096, ("normal", "peaked", "ties")), (32000, ("normal",))):
        for kind in kinds:
            lg = rng.standard_normal(V).astype(np.float32) * np.float32(2.5)
            if kind == "peaked":
                lg *= np.float32(4.0)
            if kind == "ties":
                lg = np.round(lg).astype(np.float32)
            hist = rng.integers(0, V, size=200).astype(np.int32)
            if V > 400:
                hist[60:70] = 220                                  # a whitespace id inside the penalty window
            r = len(rows)
            out[f"logits.{r}"], out[f"history.{r}"] = lg, hist
            res = []
            for top_k, top_p, penalty in configs:
                x = ref.apply_repetition_penalty(mx.array(lg.tolist()), hist.tolist(), penalty, whitespace_ids=set(ws))
                pen = np.asarray(_raw(x), np.float32).copy()
                x = ref.apply_top_k(x, min(top_k, V))
                x = ref.apply_top_p(x, top_p)
                filt = np.asarray(_raw(x), np.float32)
                kept = np.isfinite(filt)
                assert (filt[kept] == pen[kept]).all() and kept.any()
                thr = float(filt[kept].min())
                assert int((pen >= thr).sum()) == int(kept.sum())             # the kept set is a threshold on the penalised logits
                greedy = ref.sample_token(mx.array(pen.tolist()), 0.0)        # greedy decoding looks at the penalised logits
                changed = np.nonzero(pen != lg)[0].astype(np.int32)
                out[f"pen_ids.{r}.{len(res)}"], out[f"pen_vals.{r}.{len(res)}"] = changed, pen[changed]
                res.append((thr if kept.sum() < V else -np.inf, int(kept.sum()), greedy))
            out[f"results.{r}"] = np.asarray(res, np.float64)          # rows of (threshold, kept count, greedy id) per config
            rows.append((V, kind))
    out["n_rows"] = np.asarray(len(rows))
    path = os.path.join(HERE, "sampler_reference_rules.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {len(rows)} logits rows x {len(configs)} configurations to {path} ({os.path.getsize(path) / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
