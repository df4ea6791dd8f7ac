"""Training driver around the device-resident engine: the step loop of the reference's ``Trainer::train``
(cpp/src/Trainer.cpp:172-420) with its learning-rate schedule (``:40-51``), ``metrics.csv`` (``:247-255, 347-365``),
checkpoint cadence / pruning / auto-resume (``:205-245, 380-420``) and the ``Checkpoint::save/load`` file pair
(cpp/src/Checkpoint.cpp:721-1116).  File formats, the schedule and the metrics rows are produced by the native
library (csrc/checkpoint.cpp); this module only sequences the calls.

The reference's step is: get a batch, forward, loss, zero the gradients, backward, AdamW, read the loss, log.
Here the whole step is one call into the engine (``train_step_host``): ids go up, the loss comes back, nothing
else crosses the PCIe bus.
"""
from __future__ import annotations

import ctypes as C
import os
import re
import resource
import time
from dataclasses import dataclass

import numpy as np

from . import bridge

_CKPT_RE = re.compile(r"^step_(\d+)\.safetensors$")


@dataclass
class TrainerConfig:
    """Mirrors ``TrainerConfig`` (cpp/include/Trainer.hpp:26-38), same defaults."""
    max_steps: int = 100
    warmup_steps: int = 10
    lr_max: float = 3e-4
    lr_min: float = 3e-5
    log_interval: int = 10
    checkpoint_dir: str = "checkpoints"
    metrics_filepath: str = "metrics.csv"
    checkpoint_interval: int = 500
    keep_last_n_checkpoints: int = 3
    resume: bool = True
    # AdamW hyper-parameters (cpp/include/Optimizer.hpp:86-88 defaults are overridden by the trainer binary)
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    peak_flops: float = 28.3e12   # denominator of the mfu_pct column (cpp/src/Trainer.cpp:344); set to the GPU's peak


def _cfg_struct(shape) -> bridge.ModelConfig:
    return bridge.ModelConfig(shape.V, shape.H, shape.I, shape.L, shape.nH, shape.nKV, shape.hd, shape.S, shape.rope_base, shape.eps)


def scheduled_lr(step: int, cfg: TrainerConfig) -> float:
    """``Trainer::get_scheduled_lr`` (cpp/src/Trainer.cpp:40-51)."""
    return float(bridge.load_library().b200_scheduled_lr(step, cfg.warmup_steps, cfg.max_steps, cfg.lr_max, cfg.lr_min))


def _check(rc: int):
    if rc != 0:
        raise bridge.B200Error(bridge.load_library().b200_checkpoint_last_error().decode() or f"error {rc}")


# ---- checkpoints on flat host arrays (no GPU involved) ------------------------------------------------
def write_checkpoint_flat(shape, path: str, params: np.ndarray, adam_m=None, adam_v=None, step: int = 0):
    lib = bridge.load_library()
    mc = _cfg_struct(shape)
    n = int(lib.b200_checkpoint_param_count(C.byref(mc)))
    params = np.ascontiguousarray(params, np.float32)
    assert params.size == n, (params.size, n)
    mp = vp = None
    if adam_m is not None:
        adam_m, adam_v = np.ascontiguousarray(adam_m, np.float32), np.ascontiguousarray(adam_v, np.float32)
        assert adam_m.size == n and adam_v.size == n
        mp, vp = bridge._np_ptr(adam_m), bridge._np_ptr(adam_v)
    _check(lib.b200_checkpoint_write_flat(C.byref(mc), bridge._np_ptr(params), mp, vp, int(step), path.encode()))


def read_checkpoint_flat(shape, path: str, with_optimizer: bool = True):
    """-> (params, m, v, step, has_opt_state); m/v are None without ``with_optimizer``."""
    lib = bridge.load_library()
    mc = _cfg_struct(shape)
    n = int(lib.b200_checkpoint_param_count(C.byref(mc)))
    params = np.empty(n, np.float32)
    m = np.empty(n, np.float32) if with_optimizer else None
    v = np.empty(n, np.float32) if with_optimizer else None
    step, has = C.c_uint64(0), C.c_int(0)
    _check(lib.b200_checkpoint_read_flat(C.byref(mc), path.encode(), bridge._np_ptr(params),
                                         bridge._np_ptr(m) if with_optimizer else None,
                                         bridge._np_ptr(v) if with_optimizer else None, C.byref(step), C.byref(has)))
    return params, m, v, int(step.value), bool(has.value)


# ---- checkpoints of the device-resident engine ----------------------------------------------------------
def save_checkpoint(model: "bridge.Model", path: str, step: int | None = None, with_optimizer: bool = True):
    """``Checkpoint::save(path, model, optimizer, step)``; ``step=None`` stores the optimizer's own count."""
    lib = bridge.load_library()
    rc = lib.b200_checkpoint_save(model.h, path.encode(), (1 << 64) - 1 if step is None else int(step), int(with_optimizer))
    if rc:
        raise bridge.B200Error(lib.b200_checkpoint_last_error().decode() or model.ctx.lib.b200_last_error(model.ctx.h).decode())


def load_checkpoint(model: "bridge.Model", path: str, with_optimizer: bool = True) -> int:
    """``Checkpoint::load``; returns the optimizer step stored with the checkpoint (0 without optimizer state)."""
    lib = bridge.load_library()
    step = C.c_uint64(0)
    rc = lib.b200_checkpoint_load(model.h, path.encode(), int(with_optimizer), C.byref(step))
    if rc:
        raise bridge.B200Error(lib.b200_checkpoint_last_error().decode() or model.ctx.lib.b200_last_error(model.ctx.h).decode())
    return int(step.value)


def latest_checkpoint(directory: str):
    """(step, path) of the newest ``step_NNNNNNN.safetensors`` (cpp/src/Trainer.cpp:208-232), or None."""
    best = None
    if os.path.isdir(directory):
        for fn in os.listdir(directory):
            mt = _CKPT_RE.match(fn)
            if mt and (best is None or int(mt.group(1)) > best[0]):
                best = (int(mt.group(1)), os.path.join(directory, fn))
    return best if best and best[0] > 0 else None


def prune_checkpoints(directory: str, keep_last_n: int):
    """Keep the newest ``keep_last_n`` checkpoints and drop the rest with their optimizer files (``:389-420``)."""
    if keep_last_n <= 0 or not os.path.isdir(directory):
        return
    found = sorted((int(m.group(1)), os.path.join(directory, fn)) for fn in os.listdir(directory) if (m := _CKPT_RE.match(fn)))
    for _, path in found[:max(0, len(found) - keep_last_n)]:
        for p in (path, path.replace(".safetensors", ".opt.safetensors")):
            if os.path.exists(p):
                os.remove(p)


class Trainer:
    """``Trainer(config, model, optimizer, data_loader, rope)``: the optimizer and the RoPE tables live inside the
    engine; ``data_loader`` needs ``get_batch() -> int array [B, S+1] or None`` and ``skip_sequences(n)``
    (DataIngestion, cpp/include/DataIngestion.hpp)."""

    def __init__(self, config: TrainerConfig, model: "bridge.Model", data_loader):
        self.cfg, self.model, self.data = config, model, data_loader
        self.lib = bridge.load_library()

    def train(self, log=print) -> int:
        cfg, model = self.cfg, self.model
        start_step = 0
        if cfg.resume:
            found = latest_checkpoint(cfg.checkpoint_dir)
            if found:
                try:
                    start_step = load_checkpoint(model, found[1])
                    log(f"[INFO] Resumed from {found[1]}; start_step = {start_step}")
                except bridge.B200Error as e:          # the reference starts from scratch on a bad checkpoint
                    log(f"[WARNING] Failed to load checkpoint ({e}). Starting training from scratch.")
                    start_step = 0
        batch_size = getattr(self.data, "batch_size", None)
        if start_step > 0 and batch_size:
            self.data.skip_sequences(start_step * batch_size)
        _check(self.lib.b200_metrics_begin(cfg.metrics_filepath.encode(), start_step))
        shape = model.cfg
        n_params = model.n_params
        step = start_step
        for step in range(start_step, cfg.max_steps):
            t0 = time.perf_counter()
            batch = self.data.get_batch()
            if batch is None or len(batch) == 0:
                log("[INFO] End of token stream reached. Stopping training.")
                break
            batch = np.asarray(batch, np.int32)
            tokens, targets = np.ascontiguousarray(batch[:, :-1]), np.ascontiguousarray(batch[:, 1:])
            lr = scheduled_lr(step, cfg)
            n0 = model.ctx.launch_count()
            loss = model.train_step_host(tokens, targets, lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay)
            step_ms = (time.perf_counter() - t0) * 1e3
            # the reference counts seq_len = S+1 ids per sequence (cpp/src/Trainer.cpp:327)
            toks = batch.shape[0] * batch.shape[1]
            tok_s = toks / (step_ms / 1e3)
            vram_gb = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss * 1024 / 2**30
            mfu = 6.0 * n_params * toks / (step_ms / 1e3) / cfg.peak_flops * 100.0
            _check(self.lib.b200_metrics_append(cfg.metrics_filepath.encode(), step, loss, tok_s, lr, vram_gb, mfu, step_ms,
                                                model.ctx.launch_count() - n0, step_ms, 0, 0.0, 100.0))
            if step % cfg.log_interval == 0 or step == cfg.max_steps - 1:
                log(f"  Step {step:4d} | Loss: {loss:.5f} | LR: {lr:.4e} | Latency: {step_ms:.2f} ms | MFU: {mfu:.2f}%")
            if (step + 1) % cfg.checkpoint_interval == 0 or step + 1 == cfg.max_steps:
                os.makedirs(cfg.checkpoint_dir, exist_ok=True)
                save_checkpoint(model, os.path.join(cfg.checkpoint_dir, f"step_{step + 1:07d}.safetensors"))   # stores the optimizer's own step count, as the reference does
                prune_checkpoints(cfg.checkpoint_dir, cfg.keep_last_n_checkpoints)
        return step
