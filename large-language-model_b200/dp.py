"""Host-side plumbing of the data-parallel step (one process per GPU).

The reference is single-device; data parallelism is this backend's addition.  The batch is split
across replicas (independent sequences, nothing in the block couples them), every replica holds the
full weights and optimizer state, and the only exchange is the average of the fp32 gradients, which
the engine issues itself over NCCL while backward is still running (csrc/model.cu).  What is left
for the host, and lives here, is control plane over ``torch.distributed`` (any backend; gloo is enough):
passing the NCCL unique id from rank 0, picking each rank's slice of the global batch, and reducing
timings.  Keeping it free of CUDA lets world_size > 1 be tested on CPU.
"""
from __future__ import annotations

import os

import numpy as np


def env_rank_world():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def init_control_plane(backend: str = "gloo"):
    """Joins the torch.distributed group described by the torchrun environment (no-op for one rank)."""
    import torch.distributed as dist
    rank, world, _ = env_rank_world()
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend, rank=rank, world_size=world)
    return rank, world


def broadcast_bytes(payload: bytes | None, src: int = 0) -> bytes:
    """Rank ``src`` supplies ``payload`` (e.g. the 128-byte NCCL unique id); every rank returns it."""
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size() == 1:
        assert payload is not None
        return payload
    box = [payload if dist.get_rank() == src else None]
    dist.broadcast_object_list(box, src=src)
    return box[0]


def shard_batch(global_batch: np.ndarray, rank: int, world: int) -> np.ndarray:
    """Contiguous, equal slice of the leading (sequence) dimension for this rank.
    The mean loss over the global batch equals the mean of the per-rank mean losses only when the
    slices are equal, so an uneven split is refused."""
    n = global_batch.shape[0]
    if n % world:
        raise ValueError(f"global batch of {n} sequences does not split evenly over {world} replicas")
    per = n // world
    return np.ascontiguousarray(global_batch[rank * per:(rank + 1) * per])


def max_over_ranks(values):
    """Element-wise maximum over ranks of a short list of floats (timings)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def average_over_ranks(array: np.ndarray) -> np.ndarray:
    """CPU model of the engine's gradient exchange (sum over ranks / world), used by the tests."""
    import torch
    import torch.distributed as dist
    t = torch.from_numpy(np.ascontiguousarray(array, np.float64).copy())
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        t /= dist.get_world_size()
    return t.numpy()
