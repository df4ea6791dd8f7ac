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


class Membership:
    """Agreement on who takes part in the next step, reached on the host BEFORE anything is launched.

    A data-parallel step contains collectives; a rank that enters one without its peers hangs until a timeout.
    So a rank never finds out about a departure inside a collective: at every step boundary each live rank posts
    its intent for the next step ("go" or "leave") in a key-value store and reads the intents of the others.  A
    rank that leaves does so only at such a boundary, with none of its kernels or collectives in flight; a rank
    that died without a word simply never posts, and the others give up on it after ``timeout_s``.  All ranks
    therefore hold the same list of live ranks before their next launch, and the survivors can rebuild their
    communicator (or stop) instead of blocking.  Works with any ``torch.distributed`` store (TCPStore, FileStore).
    """

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, timeout_s
        self.live = list(range(world))

    def _key(self, step: int, rank: int) -> str:
        return f"membership/{step}/{rank}"

    def post(self, step: int, leaving: bool = False):
        self.store.set(self._key(step, self.rank), b"leave" if leaving else b"go")

    def agree(self, step: int, leaving: bool = False):
        """Posts this rank's intent for ``step`` and returns the sorted list of ranks that will run it."""
        import datetime
        self.post(step, leaving)
        staying = []
        for r in self.live:
            if r == self.rank:
                if not leaving:
                    staying.append(r)
                continue
            try:
                self.store.wait([self._key(step, r)], datetime.timedelta(seconds=self.timeout_s))
                if bytes(self.store.get(self._key(step, r))) == b"go":
                    staying.append(r)
            except Exception:       # noqa: BLE001 - a store timeout: the peer never posted, treat it as gone
                pass
        self.live = sorted(staying)
        return self.live
