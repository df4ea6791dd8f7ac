"""The training driver on the GPU: step loop with the reference's schedule, metrics file and checkpoint cadence
(cpp/src/Trainer.cpp:172-420); a run that is interrupted and resumed from its checkpoint must land where the
uninterrupted run lands; checkpoints of the device-resident engine round-trip weights, AdamW moments and step."""
import csv
import os

import numpy as np
import pytest

from gpu_util import bridge, ctx, rel, synth  # noqa: F401
import importlib

trainer = importlib.import_module("large-language-model_b200.trainer")

pytestmark = pytest.mark.gpu
SHAPE = dict(B=2, S=16, H=64, I=96, nH=4, nKV=2, hd=16, V=128, L=2)


class Loader:
    """Stand-in for DataIngestion (cpp/src/DataIngestion.cpp:60-83): sequences of S+1 ids, batch by batch."""

    def __init__(self, n_batches, batch_size, seq_len, vocab, seed=3):
        self.batch_size = batch_size
        self.seqs = synth.token_ids(seed, "stream", (n_batches * batch_size, seq_len + 1), vocab)
        self.i = 0

    def get_batch(self):
        b = self.seqs[self.i:self.i + self.batch_size]
        self.i += len(b)
        return b if len(b) else None

    def skip_sequences(self, n):
        self.i += min(n, len(self.seqs) - self.i)


def fresh_model(ctx, dtype="f32"):
    m = bridge.Model(ctx, bridge.Shape(**SHAPE), dtype)
    m.init_synthetic(11, 0.05)
    return m


def rows(path):
    with open(path) as f:
        return list(csv.DictReader(f))


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_interrupted_and_resumed_run_equals_the_uninterrupted_one(ctx, tmp_path, dtype):
    def cfg(tag):
        return trainer.TrainerConfig(max_steps=9, warmup_steps=3, lr_max=1e-2, lr_min=1e-3, log_interval=100,
                                     checkpoint_dir=str(tmp_path / tag / "ckpt"), metrics_filepath=str(tmp_path / tag / "metrics.csv"),
                                     checkpoint_interval=3, keep_last_n_checkpoints=2, resume=True)

    for tag in ("whole", "parts"):
        os.makedirs(tmp_path / tag)
    # uninterrupted: 9 steps
    m = fresh_model(ctx, dtype)
    trainer.Trainer(cfg("whole"), m, Loader(9, SHAPE["B"], SHAPE["S"], SHAPE["V"])).train(log=lambda s: None)
    whole_params, whole_rows = m.read_params(), rows(cfg("whole").metrics_filepath)
    m.close()
    assert [int(r["step"]) for r in whole_rows] == list(range(9))
    lrs = [trainer.scheduled_lr(s, cfg("whole")) for s in range(9)]
    np.testing.assert_allclose([float(r["learning_rate"]) for r in whole_rows], lrs, rtol=1e-5)
    assert all(np.isfinite(float(r["train_loss"])) and float(r["train_loss"]) > 0 for r in whole_rows)
    assert sorted(os.listdir(cfg("whole").checkpoint_dir)) == ["step_0000006.opt.safetensors", "step_0000006.safetensors",
                                                                "step_0000009.opt.safetensors", "step_0000009.safetensors"]
    # the stream ends after 6 batches; a new process-like start (fresh model, fresh loader) resumes from step_6
    m = fresh_model(ctx, dtype)
    last = trainer.Trainer(cfg("parts"), m, Loader(6, SHAPE["B"], SHAPE["S"], SHAPE["V"])).train(log=lambda s: None)
    m.close()
    assert last == 6 and len(rows(cfg("parts").metrics_filepath)) == 6
    m = bridge.Model(ctx, bridge.Shape(**SHAPE), dtype)
    m.init_synthetic(999, 0.05)                                  # different weights: the checkpoint must replace them
    trainer.Trainer(cfg("parts"), m, Loader(9, SHAPE["B"], SHAPE["S"], SHAPE["V"])).train(log=lambda s: None)
    parts_params, parts_rows = m.read_params(), rows(cfg("parts").metrics_filepath)
    m.close()
    assert [int(r["step"]) for r in parts_rows] == list(range(9))
    tol = 2e-4 if dtype == "f32" else 2e-3      # atomically accumulated gradients are not bit-reproducible and AdamW amplifies the noise; a wrong resume is off by >1e-2
    assert rel(parts_params, whole_params) < tol
    np.testing.assert_allclose([float(r["train_loss"]) for r in parts_rows], [float(r["train_loss"]) for r in whole_rows], rtol=10 * tol)


def test_engine_checkpoint_round_trip(ctx, tmp_path):
    m = fresh_model(ctx, "bf16")
    tok = synth.token_ids(5, "t", (SHAPE["B"], SHAPE["S"] + 1), SHAPE["V"])
    for _ in range(3):
        m.train_step_host(np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:]), 1e-2)
    path = str(tmp_path / "step_0000003.safetensors")
    trainer.save_checkpoint(m, path)
    p, mm, vv, step, has = trainer.read_checkpoint_flat(bridge.Shape(**SHAPE), path)
    em, ev, estep = m.read_opt_state()
    assert has and step == 3 == estep
    np.testing.assert_array_equal(p, m.read_params())
    np.testing.assert_array_equal(mm, em)
    np.testing.assert_array_equal(vv, ev)
    assert np.abs(mm).max() > 0 and vv.min() >= 0
    other = bridge.Model(ctx, bridge.Shape(**SHAPE), "bf16")
    other.init_synthetic(1, 0.02)
    assert trainer.load_checkpoint(other, path) == 3
    np.testing.assert_array_equal(other.read_params(), p)
    om, ov, ostep = other.read_opt_state()
    np.testing.assert_array_equal(om, em); np.testing.assert_array_equal(ov, ev)
    assert ostep == 3
    # both continue identically
    a = m.train_step_host(np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:]), 1e-2)
    b = other.train_step_host(np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:]), 1e-2)
    assert abs(a - b) <= 2e-3 * abs(a)
    m.close(); other.close()


def test_optimizer_in_backward_order_gives_the_same_update(ctx, monkeypatch):
    """B200_FUSED_OPT=1 runs each bucket's AdamW on a side stream during the backward pass; same result."""
    tok = synth.token_ids(6, "t", (SHAPE["B"], SHAPE["S"] + 1), SHAPE["V"])
    x, y = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
    results = []
    for flag in ("0", "1"):
        monkeypatch.setenv("B200_FUSED_OPT", flag)
        m = fresh_model(ctx, "bf16")
        losses = [m.train_step_host(x, y, 1e-2) for _ in range(4)]
        results.append((losses, m.read_params(), m.read_opt_state()))
        m.close()
    (l0, p0, (m0, v0, s0)), (l1, p1, (m1, v1, s1)) = results
    assert s0 == s1 == 4
    # Gradients are not bit-reproducible between runs (fp32 atomics in the embedding and attention gradients) and AdamW
    # normalises them: a gradient near zero can flip its sign and move that weight by a whole lr step, and its moments
    # with it.  So the check counts elements instead of taking a norm: a bucket that missed or doubled one of the four
    # updates would move EVERY weight of the bucket (>= 5 % of the model) by about lr and its moments by about a quarter.
    lr = 1e-2
    np.testing.assert_allclose(l0, l1, rtol=5e-3)
    moved = np.mean(np.abs(p1 - p0) > 0.25 * lr)
    # (bf16 activations turn a reordered fp32 sum into an occasional different rounding, so moments of typical size agree
    # to a fraction of a percent while those near zero can be off by more than their own size: hence the absolute floor)
    rms = lambda a: float(np.sqrt(np.mean(np.square(a, dtype=np.float64))))
    m_off = np.mean(np.abs(m1 - m0) > 0.1 * np.abs(m0) + 0.05 * rms(m0))
    v_off = np.mean(np.abs(v1 - v0) > 0.1 * np.abs(v0) + 0.05 * rms(v0))
    assert moved < 0.01 and m_off < 0.01 and v_off < 0.01, (moved, m_off, v_off)
