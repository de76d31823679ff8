"""Failure detection on the host, with gloo ranks on CPU and no GPU involved: a rank that never
reaches a step is named before anything is launched for that step; a rank that never enters a
collective makes the others' call end with an error at the process group's deadline instead of
hanging; a slab that does not match its rank's column range is refused before the collective."""
import datetime
import os
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lost_rank_worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    from nnabla_b200 import sharding
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    guard = sharding.StepGuard(store, rank, world, timeout_s=2.0)
    guard.arrive("step0")          # everybody is there
    out = {"step0": True}
    if rank == world - 1:
        # this rank leaves between the steps (nothing of it is in flight); it stays alive until the
        # others have noticed, so that their store connection is not what fails
        store.wait(["noticed"], datetime.timedelta(seconds=30))
        results[rank] = out
        return
    t0 = time.monotonic()
    try:
        guard.arrive("step1")
        out["step1"] = "arrived"
    except sharding.PeerLost as e:
        out["step1"] = ("lost", e.missing, time.monotonic() - t0)
    if rank == 0:
        time.sleep(0.5)
        store.set("noticed", b"1")
    results[rank] = out


def test_a_rank_that_leaves_is_named_before_the_next_launch():
    port = 29700 + os.getpid() % 200
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_lost_rank_worker, args=(3, port, results), nprocs=3, join=True)
    for r in (0, 1):
        kind, missing, waited = results[r]["step1"]
        assert kind == "lost" and missing == [2] and waited < 10.0
    assert results[2] == {"step0": True}


def _stuck_collective_worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    from nnabla_b200 import sharding
    y = torch.ones(4, 3) * rank
    full = sharding.gather_columns(y, 6)          # a step every rank takes part in
    ok = bool(torch.equal(full[:, 3:], torch.ones(4, 3)))
    if rank == 1:
        time.sleep(8)                             # never enters the second collective
        results[rank] = ("skipped", ok)
        return
    t0 = time.monotonic()
    try:
        sharding.gather_columns(y, 6)
        results[rank] = ("returned", ok)
    except RuntimeError as e:
        results[rank] = ("error", ok, time.monotonic() - t0, str(e)[:80])


def test_a_collective_a_rank_never_enters_ends_with_an_error():
    port = 29900 + os.getpid() % 90
    mgr = mp.Manager()
    results = mgr.dict()
    try:
        mp.spawn(_stuck_collective_worker, args=(2, port, results), nprocs=2, join=True)
    except Exception:  # noqa: BLE001 - a rank whose process group was torn down may exit non-zero
        pass
    assert results[0][0] == "error" and results[0][1] is True and results[0][2] < 7.5
    assert results[1] == ("skipped", True)


def test_mismatched_slab_is_refused_before_the_collective():
    sys.path.insert(0, ROOT)
    from nnabla_b200 import sharding
    store = dist.HashStore()
    dist.init_process_group("gloo", store=store, rank=0, world_size=1)
    try:
        with pytest.raises(ValueError, match="slab width"):
            sharding.gather_columns(torch.zeros(4, 5), 6)   # this rank owns 6 columns, not 5
        with pytest.raises(ValueError, match="bad rank"):
            sharding.shard_range(6, 2, 2)
    finally:
        dist.destroy_process_group()
