"""Batch sharding of the embedding forward over the GPUs of one node.

The reference has no multi-GPU path for this model: its served trunk runs one sequence per forward with the batch axis
fixed at 1 (``emmy/serving/ARCHITECTURE.md:93-123``) and its only multi-GPU code pins autotune subprocesses to devices
(``emmy/compiler/backend/cuda/program.py:1415-1430``). Sequences are independent end to end, so the batch is split
into contiguous shards, one process per GPU with replicated weights, and the only exchange is one all-gather of the
pooled embeddings (``[batch/world, hidden]`` fp32 per rank) over NCCL. No kernel reads a peer's memory.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    start: int
    stop: int

    @property
    def size(self) -> int:
        return self.stop - self.start


def shard_batch(total: int, rank: int, world: int) -> Shard:
    """Contiguous shard of ``total`` sequences for ``rank``: the first ``total % world`` ranks get one extra."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    if total < 0:
        raise ValueError("total must be non-negative")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return Shard(rank, world, start, start + base + (1 if rank < extra else 0))


def env_rank_world() -> tuple[int, int, int]:
    """(rank, local_rank, world) from the torchrun environment; (0, 0, 1) when not launched by it."""
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def init_process_group(backend: str | None = None) -> tuple[int, int, int]:
    """Join the job's process group (NCCL on GPUs, gloo otherwise). Rendezvous comes from MASTER_ADDR/MASTER_PORT."""
    rank, local_rank, world = env_rank_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, local_rank, world


def gather_embeddings(local: torch.Tensor, total: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather the per-rank pooled embeddings into ``[total, hidden]`` in shard order. Equal shards use one
    ``all_gather_into_tensor``; ragged shards fall back to a padded gather."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        if out is not None:
            out.copy_(local)
            return out
        return local
    world = dist.get_world_size()
    hidden = local.shape[-1]
    if out is None:
        out = torch.empty(total, hidden, dtype=local.dtype, device=local.device)
    if total % world == 0:
        dist.all_gather_into_tensor(out, local.contiguous())
        return out
    width = (total + world - 1) // world
    padded = torch.zeros(width, hidden, dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    buf = torch.empty(world * width, hidden, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, padded)
    for r in range(world):
        sh = shard_batch(total, r, world)
        out[sh.start: sh.stop] = buf[r * width: r * width + sh.size]
    return out


class PipelinedGather:
    """All-gather of the pooled embeddings that does not stall the next forward.

    A forward's last kernel writes ``[batch/world, hidden]`` embeddings; gathering them on the compute stream makes
    every rank wait for the slowest one at every step before its next forward may start. Here the shard is copied to
    one of ``depth`` staging buffers (compute stream, 32 KB) and gathered from there with an asynchronous NCCL
    all-gather: the next forward starts at once, and a buffer is reused only after the gather that read it has
    completed (a stream-level wait on a collective issued ``depth`` steps earlier, long done). :meth:`result` waits
    for the most recent gather and returns its ``[total, hidden]`` output. Equal shards only."""

    def __init__(self, shard_rows: int, total: int, hidden: int, device, dtype=torch.float32, depth: int = 2) -> None:
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        if shard_rows * self.world != total:
            raise ValueError("PipelinedGather needs equal shards (total = world * shard rows)")
        self.stage = [torch.empty(shard_rows, hidden, dtype=dtype, device=device) for _ in range(depth)]
        self.out = [torch.empty(total, hidden, dtype=dtype, device=device) for _ in range(depth)]
        self.work: list = [None] * depth
        self.n = 0

    def submit(self, local: torch.Tensor) -> None:
        k = self.n % len(self.stage)
        if self.work[k] is not None:
            self.work[k].wait()          # the gather that last used this pair of buffers (stream-level for NCCL)
            self.work[k] = None
        self.stage[k].copy_(local)
        if self.world > 1:
            self.work[k] = dist.all_gather_into_tensor(self.out[k], self.stage[k], async_op=True)
        else:
            self.out[k].copy_(self.stage[k])
        self.n += 1

    def result(self) -> torch.Tensor:
        """The gathered embeddings of the most recent :meth:`submit` (the current stream waits for that gather)."""
        if self.n == 0:
            raise RuntimeError("nothing has been submitted")
        k = (self.n - 1) % len(self.stage)
        if self.work[k] is not None:
            self.work[k].wait()
            self.work[k] = None
        return self.out[k]

    def flush(self) -> None:
        """Make the current stream wait for every gather still in flight."""
        for k, w in enumerate(self.work):
            if w is not None:
                w.wait()
                self.work[k] = None
