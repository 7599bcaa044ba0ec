"""World-size-2 data-parallel path on CPU (gloo): shards, per-rank execution with a fake
executor in place of the GPU graph, and the ordered gather."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_infer(images, tokens, noise):
    # deterministic per-observation "action chunk": depends only on that observation
    return (noise * 2.0 + images.reshape(images.shape[0], -1).sum(axis=1, dtype=np.int64)
            .astype(np.float32)[:, None, None] * 1e-6 + tokens.sum(axis=1)[:, None, None] * 1e-3
            ).astype(np.float32)


def _worker(rank, world, port, batch, result_dir):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    from apxinf_b200.parallel import run_sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(5)
    images = rng.integers(0, 256, size=(batch, 2, 4, 4, 3), dtype=np.uint8)
    tokens = rng.integers(0, 100, size=(batch, 3)).astype(np.uint32)
    noise = rng.standard_normal((batch, 5, 8)).astype(np.float32)
    out, shard = run_sharded(_fake_infer, images, tokens, noise, rank, world, gather=True, dist=dist)
    np.save(os.path.join(result_dir, f"out_{rank}.npy"), out)
    np.save(os.path.join(result_dir, f"shard_{rank}.npy"), np.array([shard.start, shard.stop]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("batch", [7, 2, 1])
def test_two_rank_sharded_run_matches_single_process(tmp_path, batch):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, batch, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(5)
    images = rng.integers(0, 256, size=(batch, 2, 4, 4, 3), dtype=np.uint8)
    tokens = rng.integers(0, 100, size=(batch, 3)).astype(np.uint32)
    noise = rng.standard_normal((batch, 5, 8)).astype(np.float32)
    want = _fake_infer(images, tokens, noise)
    bounds = []
    for rank in range(world):
        got = np.load(tmp_path / f"out_{rank}.npy")
        assert np.array_equal(got, want)
        bounds.append(tuple(np.load(tmp_path / f"shard_{rank}.npy")))
    assert bounds[0][0] == 0 and bounds[0][1] == bounds[1][0] and bounds[1][1] == batch
