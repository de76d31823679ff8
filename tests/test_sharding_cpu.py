"""Host-side sharding logic with world_size-2 gloo ranks on CPU: column-sharded
affine with per-shard alpha reproduces the unsharded oracle result after the
gather; batch shards gather back in order; ragged splits."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nnabla_b200 import sharding
        from oracle import oracle
        rng = np.random.RandomState(0)  # same seed on every rank: x is replicated without a broadcast
        x = rng.randn(6, 16).astype(np.float32)
        w = (0.02 * rng.randn(16, 11)).astype(np.float32)  # 11 columns: ragged over 2 ranks
        b = rng.randn(11).astype(np.float32)
        ws, bs, (c0, c1) = sharding.column_shard(torch.from_numpy(w), torch.from_numpy(b), rank, world)
        ys, wbs, als = oracle.binary_weight_affine(x, ws.numpy(), bs.numpy())
        full = sharding.gather_columns(torch.from_numpy(ys), 11)
        want, _, wal = oracle.binary_weight_affine(x, w, b)
        ok_cols = np.array_equal(full.numpy(), want) and np.array_equal(als, wal[c0:c1])
        imgs = torch.arange(5 * 3, dtype=torch.float32).reshape(5, 3)
        mine = sharding.batch_shard(imgs, rank, world)
        back = sharding.gather_batch(mine * 2, 5)
        ok_batch = torch.equal(back, imgs * 2)
        results[rank] = (ok_cols, ok_batch, (c0, c1))
    finally:
        dist.destroy_process_group()


def test_shard_range():
    from nnabla_b200.sharding import shard_range
    assert [shard_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [shard_range(8192, r, 8) for r in range(8)][-1] == (7168, 8192)
    assert shard_range(1, 1, 2) == (1, 1)
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_column_and_batch_sharding_two_ranks():
    port = 29500 + os.getpid() % 1000
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert results[0][:2] == (True, True) and results[1][:2] == (True, True)
    assert results[0][2] == (0, 6) and results[1][2] == (6, 11)
