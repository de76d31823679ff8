"""The data-parallel communicator with world_size-2 gloo ranks on CPU: every
collective of nnabla's Communicator interface (include/nbla/communicator.hpp)
with packed (inplace=False) and per-array (inplace=True) transfers, division,
named groups and the bucketed gradient all-reduce."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from nnabla_b200 import communicators as C
    comm = C.MultiProcessDataParallelCommunicator()
    ok = {}
    try:
        with pytest.raises(RuntimeError):
            comm.size
        comm.init("gloo")
        ok["identity"] = (comm.size, comm.rank, comm.local_rank) == (world, rank, rank)
        with pytest.raises(RuntimeError):
            comm.init("gloo")
        # all_reduce: packed and in place, with and without division
        for inplace in (False, True):
            a = [torch.full((3, 2), float(rank + 1)), torch.arange(5, dtype=torch.float32) * (rank + 1)]
            comm.all_reduce(a, division=False, inplace=inplace)
            ok["all_reduce_%d" % inplace] = bool(torch.equal(a[0], torch.full((3, 2), 3.0)) and
                                                 torch.equal(a[1], torch.arange(5, dtype=torch.float32) * 3))
            b = torch.full((4,), float(rank + 1))
            comm.all_reduce(b, division=True, inplace=inplace)
            ok["all_reduce_div_%d" % inplace] = bool(torch.equal(b, torch.full((4,), 1.5)))
        # reduce: only dst changes
        c = torch.full((3,), float(rank + 1))
        comm.reduce(c, 1, division=True)
        ok["reduce"] = bool(torch.equal(c, torch.full((3,), 1.5 if rank == 1 else 1.0)))
        # bcast
        d = [torch.full((2,), float(rank)), torch.full((3,), float(rank) + 10)]
        comm.bcast(d, 1)
        ok["bcast"] = bool(torch.equal(d[0], torch.full((2,), 1.0)) and torch.equal(d[1], torch.full((3,), 11.0)))
        # all_gather
        out = [torch.zeros(2), torch.zeros(2)]
        comm.all_gather(torch.full((2,), float(rank + 5)), out)
        ok["all_gather"] = bool(torch.equal(out[0], torch.full((2,), 5.0)) and torch.equal(out[1], torch.full((2,), 6.0)))
        # reduce_scatter
        pieces = [torch.full((2,), float(rank + 1) * (p + 1)) for p in range(world)]
        mine = torch.zeros(2)
        comm.reduce_scatter(pieces, mine, division=False)
        ok["reduce_scatter"] = bool(torch.equal(mine, torch.full((2,), 3.0 * (rank + 1))))
        # groups
        comm.new_group(("solo", [0]))
        ok["groups"] = comm.find_group("solo") == [0] and comm.find_group("nobody") == [] and \
            comm.list_groups()["world"] == [0, 1]
        e = torch.full((2,), float(rank + 1))
        comm.all_reduce(e, group="solo")
        ok["group_reduce"] = bool(torch.equal(e, torch.full((2,), float(rank + 1))))  # one member: unchanged
        # bucketed gradient all-reduce
        grads = [torch.full((n,), float(rank + 1)) for n in (5, 7, 3, 11)]
        comm.all_reduce_callback(grads, pack_size=10, division=True, scale_grad=2.0)()
        ok["callback"] = all(bool(torch.equal(g, torch.full_like(g, 3.0))) for g in grads)
        comm.barrier()
        results[rank] = ok
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_communicator_two_ranks():
    port = 29800 + os.getpid() % 150
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    for r in range(2):
        assert all(results[r].values()), (r, {k: v for k, v in results[r].items() if not v})


def test_single_process_communicator_is_not_provided():
    sys.path.insert(0, ROOT)
    from nnabla_b200 import communicators as C
    with pytest.raises(NotImplementedError):
        C.DataParallelCommunicator()
