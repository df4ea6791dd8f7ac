"""Data-parallel path (more than one rank).  On CPU: world_size-2 gloo ranks check the host plumbing and
that batch sharding + gradient averaging reproduces the single-device step of the CPU checker.  On a
box with >= 2 GPUs: the engine's NCCL gradient exchange against a single-device run of the engine."""
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(mode, nproc, tmp_path, timeout):
    out = tmp_path / f"dp_{mode}.txt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "dp_worker.py"), mode, str(out)]
    env = dict(os.environ, OMP_NUM_THREADS="2", NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert out.read_text() == "OK", out.read_text()


def test_two_gloo_ranks_reproduce_the_single_device_step(tmp_path):
    _launch("cpu", 2, tmp_path, timeout=300)


def test_uneven_split_is_refused():
    import importlib
    import numpy as np
    dp = importlib.import_module("large-language-model_b200.dp")
    with pytest.raises(ValueError):
        dp.shard_batch(np.zeros((5, 3)), 0, 2)
    assert dp.shard_batch(np.arange(12).reshape(4, 3), 1, 2).tolist() == [[6, 7, 8], [9, 10, 11]]


@pytest.mark.gpu
def test_nccl_gradient_exchange_matches_single_device(tmp_path):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    _launch("gpu", 2, tmp_path, timeout=600)


@pytest.mark.parametrize("mode", ["leave", "vanish"])
def test_a_rank_that_departs_between_steps_is_noticed_on_the_host(tmp_path, mode):
    """Three gloo ranks; the last one leaves after two steps (announced, or silently).  The survivors agree on the new
    membership before their next collective and finish with a two-rank group: no rank blocks, none is killed."""
    out = tmp_path / f"dp_{mode}.txt"
    port = _free_port()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "dp_worker.py"), mode, str(out)]
    env = dict(os.environ, OMP_NUM_THREADS="1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    survivors = [tmp_path / f"dp_{mode}.txt.rank{k}" for k in (0, 1)]
    assert all(p.exists() and p.read_text() == "OK" for p in survivors), r.stdout[-2000:] + r.stderr[-4000:]
