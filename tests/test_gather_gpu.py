"""Column-sharded fixed-point affine with the gather fused into the contraction
epilogue (nb200_affine_*_gather_f32): every rank's slab must land in every
rank's [rows, N] result, bit-identical to the unsharded product and to the
oracle.

On one GPU the ranks are emulated as consecutive calls of one process that
each store into all the result matrices (no kernel waits on another, so
nothing needs to run concurrently). With two or more GPUs the same runs as
one process per GPU over matrices shared through nb200_ipc_*."""
import os
import sys

import numpy as np
import pytest
import torch

from golden_util import bits
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DX, DW = 2.0 ** -5, 2.0 ** -10


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def F():
    from nnabla_b200 import _capi, functions
    _capi.call("nb200_check_device")
    return functions


def make_case(M, K, N, seed):
    rng = np.random.RandomState(seed)
    xq = oracle.fixed_point_quantize(rng.randn(M, K).astype(np.float32), True, 8, DX)
    wq = oracle.fixed_point_quantize((0.02 * rng.randn(K, N)).astype(np.float32), True, 8, DW)
    b = (0.01 * rng.randn(N)).astype(np.float32)
    return xq, wq, b


@pytest.mark.parametrize("M,K,N,world", [(384, 512, 640, 2), (130, 256, 1001, 3), (256, 128, 2048, 8), (64, 64, 7, 1)])
def test_emulated_ranks_one_gpu(F, M, K, N, world):
    from nnabla_b200.sharding import shard_range
    xq, wq, b = make_case(M, K, N, N)
    want = oracle.affine(xq, wq, b)
    ys = [torch.full((M, N), float("nan"), device="cuda") for _ in range(world)]
    xd = dev(xq)
    for r in range(world):
        c0, c1 = shard_range(N, r, world)
        if c1 == c0:
            continue
        F.affine_fixed_point_gather(xd, dev(wq[:, c0:c1]), DX, DW, dev(b[c0:c1]), ys, r, N, c0)
    F.check_device_status()
    for r in range(world):
        assert np.array_equal(bits(ys[r].cpu().numpy()), bits(want)), "rank %d" % r


def test_emulated_ranks_from_codes(F):
    from nnabla_b200.sharding import shard_range
    M, K, N, world = 200, 384, 900, 4
    rng = np.random.RandomState(5)
    x = rng.randn(M, K).astype(np.float32)
    w = (0.02 * rng.randn(K, N)).astype(np.float32)
    _, xc = F.fixed_point_quantize_with_codes(dev(x), True, 8, DX)
    _, wc = F.fixed_point_quantize_with_codes(dev(w), True, 8, DW)
    whole = F.affine_from_codes(xc, wc, DX, DW, None)
    ys = [torch.zeros((M, N), device="cuda") for _ in range(world)]
    for r in range(world):
        c0, c1 = shard_range(N, r, world)
        F.affine_from_codes_gather(xc, wc[:, c0:c1].contiguous(), DX, DW, None, ys, r, N, c0)
    F.check_device_status()
    for y in ys:
        assert torch.equal(y, whole)


def test_gather_argument_errors(F):
    from nnabla_b200._capi import NB200Error
    xq, wq, b = make_case(32, 64, 48, 1)
    y = torch.zeros((32, 48), device="cuda")
    with pytest.raises(NB200Error):  # more ranks than one box holds
        F.affine_fixed_point_gather(dev(xq), dev(wq), DX, DW, None, [y] * 9, 0, 48, 0)
    with pytest.raises(NB200Error):  # rank outside the list
        F.affine_fixed_point_gather(dev(xq), dev(wq), DX, DW, None, [y, y], 2, 48, 0)
    with pytest.raises(NB200Error):  # slab sticks out of the result
        F.affine_fixed_point_gather(dev(xq), dev(wq), DX, DW, None, [y], 0, 48, 8)
    with pytest.raises(NB200Error):  # a null result matrix
        F.affine_fixed_point_gather(dev(xq), dev(wq), DX, DW, None, [y, 0], 0, 48, 0)


def _rank_main(rank, world, port, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nnabla_b200 import functions as Fn
        from nnabla_b200 import sharding
        M, K, N = 512, 768, 1000 + 24 * world
        xq, wq, b = make_case(M, K, N, 3)  # same seed on every rank: x is replicated without a broadcast
        want = oracle.affine(xq, wq, b)
        mats = sharding.PeerMatrices(M, N)
        mats.local.fill_(float("nan"))
        mats.fence()
        c0, c1 = sharding.shard_range(N, rank, world)
        for _ in range(2):  # a second pass overwrites the first with the same values
            Fn.affine_fixed_point_gather(dev(xq), dev(wq[:, c0:c1]), DX, DW, dev(b[c0:c1]), mats.ptrs, rank, N, c0)
            mats.fence()
        Fn.check_device_status()
        got = mats.local.cpu().numpy()
        results[rank] = bool(np.array_equal(bits(got), bits(want)))
        mats.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_per_gpu():
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 8)
    port = 29600 + os.getpid() % 300
    results = mp.Manager().dict()
    mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
    assert [results[r] for r in range(world)] == [True] * world


def _comm_main(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    from nnabla_b200 import communicators as C
    comm = C.MultiProcessDataParallelCommunicator()
    try:
        comm.init("nccl")
        dev_ = torch.device("cuda", rank)
        grads = [torch.full((n,), float(rank + 1), device=dev_) for n in (1000, 77, 4096, 5)]
        comm.all_reduce(grads, division=True, inplace=False)
        mean = sum(range(1, world + 1)) / world
        ok = all(bool(torch.allclose(g, torch.full_like(g, mean))) for g in grads)
        grads = [torch.full((n,), float(rank + 1), device=dev_) for n in (300000, 70000, 5)]
        comm.all_reduce_callback(grads, pack_size=100000, division=False)()
        ok = ok and all(bool(torch.equal(g, torch.full_like(g, float(sum(range(1, world + 1)))))) for g in grads)
        out = [torch.zeros(3, device=dev_) for _ in range(world)]
        comm.all_gather(torch.full((3,), float(rank), device=dev_), out)
        ok = ok and all(bool(torch.equal(out[r], torch.full((3,), float(r), device=dev_))) for r in range(world))
        torch.cuda.synchronize()
        results[rank] = ok
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_communicator_over_nccl():
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 8)
    port = 29650 + os.getpid() % 200
    results = mp.Manager().dict()
    mp.spawn(_comm_main, args=(world, port, results), nprocs=world, join=True)
    assert [results[r] for r in range(world)] == [True] * world
