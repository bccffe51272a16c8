"""Batch-sharded forward over two GPUs with NCCL against the single-GPU forward (skipped on a one-GPU machine)."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q) -> None:
    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from deplodock_b200.dist import gather_embeddings, init_process_group, shard_batch
    from deplodock_b200.model import EmbedForward
    from oracle import inputs

    r, local, w = init_process_group("nccl")
    cfg = inputs.EmbedModelConfig().small(layers=2, vocab=300)
    sd = inputs.embed_model_weights(cfg)
    ids = inputs.token_ids(6, 96, cfg.vocab_size, seed=3)
    sh = shard_batch(6, r, w)
    model = EmbedForward(cfg, sd, batch=sh.size, seq=96, device=f"cuda:{local}")
    got = gather_embeddings(model(ids[sh.start:sh.stop]), 6)
    torch.cuda.synchronize()
    if r == 0:
        q.put(got.cpu())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_forward_equals_single_gpu(libemk):
    from deplodock_b200.model import EmbedForward
    from oracle import inputs

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    gathered = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    cfg = inputs.EmbedModelConfig().small(layers=2, vocab=300)
    sd = inputs.embed_model_weights(cfg)
    ids = inputs.token_ids(6, 96, cfg.vocab_size, seed=3)
    single = EmbedForward(cfg, sd, batch=6, seq=96)(ids).cpu()
    assert torch.equal(gathered, single), "sequences are independent: shards must reproduce the full batch bit for bit"
