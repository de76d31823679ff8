"""Data-parallel communicator with the interface of nnabla's Communicator
(include/nbla/communicator.hpp:61-293, Python face in
python/src/nnabla/communicator.pyx:43-537) for one process per GPU.

The reference's core only declares the interface (every collective of
src/nbla/communicator/communicator.cpp raises "not implemented"); the
implementation normally comes from the CUDA extension over NCCL. Here the
collectives are torch.distributed calls (NCCL between GPUs over NVLink, gloo
between CPU ranks in the tests); arrays are torch tensors and every call
changes them in place, as the reference changes its NdArrays.

Semantics kept from the interface:
  * `division=True` divides the reduced values by the size of the group;
  * `inplace=False` packs a list of arrays into one buffer, runs ONE
    collective and unpacks (fewer launches for many small gradients),
    `inplace=True` runs one collective per array on the array itself;
  * groups are named; "world" always exists (communicator.hpp:103-117).
"""
import os

import torch
import torch.distributed as dist


def _as_list(data):
    return list(data) if isinstance(data, (list, tuple)) else [data]


class Communicator:
    def __init__(self, ctx=None):
        self.ctx = ctx
        self._groups = {}
        self._initialized = False

    # ---- identity ----------------------------------------------------------------
    @property
    def name(self):
        return "MultiProcessDataParallelCommunicator"

    @property
    def size(self):
        self._check()
        return dist.get_world_size()

    @property
    def rank(self):
        self._check()
        return dist.get_rank()

    @property
    def local_rank(self):
        self._check()
        return int(os.environ.get("LOCAL_RANK", self.rank))

    def _check(self):
        if not self._initialized:
            raise RuntimeError("Communicator is not initialized: call init() first.")

    def init(self, backend=None):
        """Joins (or creates from RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT)
        the process group. As in the reference, init() may be called once."""
        if self._initialized:
            raise RuntimeError("Communicator was already initialized.")
        if not dist.is_initialized():
            if backend is None:
                backend = "nccl" if torch.cuda.is_available() else "gloo"
            if backend == "nccl":
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
            dist.init_process_group(backend)
        self._groups = {"world": (None, list(range(dist.get_world_size())))}
        self._initialized = True

    def barrier(self):
        self._check()
        dist.barrier()

    def abort(self):
        """Leaves the job at once (the reference calls MPI_Abort)."""
        os._exit(1)

    # ---- groups --------------------------------------------------------------------
    def new_group(self, name_ranks):
        """name_ranks = (name, [ranks]); collective over all ranks. Returns the
        ranks of the group (communicator.pyx:133-155)."""
        self._check()
        name, ranks = name_ranks
        ranks = sorted(int(r) for r in ranks)
        if name in self._groups:
            raise RuntimeError("group %s already exists" % name)
        if not ranks or ranks[0] < 0 or ranks[-1] >= self.size:
            raise RuntimeError("ranks of group %s are outside the world" % name)
        self._groups[name] = (dist.new_group(ranks), ranks)
        return {name: ranks}

    def list_groups(self):
        self._check()
        return {k: v[1] for k, v in self._groups.items()}

    def find_group(self, group):
        self._check()
        return self._groups[group][1] if group in self._groups else []

    def _group(self, group):
        self._check()
        if group not in self._groups:
            raise RuntimeError("group %s does not exist" % group)
        pg, ranks = self._groups[group]
        return pg, ranks, (dist.get_rank() in ranks)

    # ---- packing ---------------------------------------------------------------------
    @staticmethod
    def _pack(arrays):
        """One flat buffer holding the arrays back to back (a single gather kernel)."""
        return torch.cat([a.reshape(-1) for a in arrays])

    @staticmethod
    def _unpack(flat, arrays):
        """Copies the flat buffer back into the arrays (one multi-tensor copy)."""
        views = [v.view_as(a) for v, a in zip(flat.split([a.numel() for a in arrays]), arrays)]
        torch._foreach_copy_(list(arrays), views)

    def _run(self, arrays, inplace, fn):
        """Applies collective `fn(tensor)` to each array (inplace) or once to the packed arrays."""
        for a in arrays:
            if not a.is_contiguous():
                raise RuntimeError("arrays must be contiguous")
        if inplace or len(arrays) == 1:
            for a in arrays:
                fn(a)
        else:
            flat = self._pack(arrays)
            fn(flat)
            self._unpack(flat, arrays)

    # ---- collectives -------------------------------------------------------------------
    def all_reduce(self, data, division=False, inplace=False, group="world"):
        """Sum over the group into every member (communicator.hpp:151-170)."""
        pg, ranks, member = self._group(group)
        if not member:
            return

        def fn(t):
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=pg)
            if division:
                t.div_(len(ranks))
        self._run(_as_list(data), inplace, fn)

    def reduce(self, data, dst, division=False, inplace=False, group="world"):
        """Sum over the group into rank `dst` (communicator.hpp:119-145); the
        arrays of the other ranks are left as they are."""
        pg, ranks, member = self._group(group)
        if not member:
            return

        def fn(t):
            keep = None if dist.get_rank() == dst else t.clone()
            dist.reduce(t, dst, op=dist.ReduceOp.SUM, group=pg)
            if keep is not None:
                t.copy_(keep)
            elif division:
                t.div_(len(ranks))
        self._run(_as_list(data), inplace, fn)

    def bcast(self, data, src, inplace=False, group="world"):
        pg, ranks, member = self._group(group)
        if not member:
            return
        self._run(_as_list(data), inplace, lambda t: dist.broadcast(t, src, group=pg))

    def all_gather(self, ndarray, ndarray_list, group="world"):
        """ndarray_list[r] receives rank r's ndarray (communicator.hpp:232-241)."""
        pg, ranks, member = self._group(group)
        if not member:
            return
        if len(ndarray_list) != len(ranks):
            raise RuntimeError("ndarray_list needs one array per rank of the group")
        dist.all_gather(list(ndarray_list), ndarray, group=pg)

    def reduce_scatter(self, ndarray_list, ndarray, division=False, group="world"):
        """ndarray receives the sum over the group of every rank's
        ndarray_list[this rank's position] (communicator.hpp:199-209)."""
        pg, ranks, member = self._group(group)
        if not member:
            return
        if len(ndarray_list) != len(ranks):
            raise RuntimeError("ndarray_list needs one array per rank of the group")
        if dist.get_backend(pg) == "gloo":  # gloo has no reduce_scatter: reduce every piece to its owner
            for pos, r in enumerate(ranks):
                piece = ndarray_list[pos].clone()
                dist.reduce(piece, r, op=dist.ReduceOp.SUM, group=pg)
                if r == dist.get_rank():
                    ndarray.copy_(piece)
        else:
            dist.reduce_scatter(ndarray, list(ndarray_list), op=dist.ReduceOp.SUM, group=pg)
        if division:
            ndarray.div_(len(ranks))

    def all_reduce_callback(self, data, pack_size, division=False, group="world", scale_grad=1.0, keep_dtype=False):
        """Gradient all-reduce in buckets of about `pack_size` values
        (communicator.hpp:172-197). The reference returns a callback that the
        graph engine fires during backward; without a graph engine the object
        returned here is called with nothing once the gradients exist and runs
        the buckets back to back as asynchronous collectives."""
        arrays = _as_list(data)
        pg, ranks, member = self._group(group)
        comm = self

        class _Callback:
            def __call__(self):
                if not member:
                    return
                buckets, cur, n = [], [], 0
                for a in arrays:
                    cur.append(a)
                    n += a.numel()
                    if n >= pack_size:
                        buckets.append(cur)
                        cur, n = [], 0
                if cur:
                    buckets.append(cur)
                pending = []
                for b in buckets:
                    flat = comm._pack(b)
                    if scale_grad != 1.0:
                        flat.mul_(scale_grad)
                    pending.append((dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=pg, async_op=True), flat, b))
                for work, flat, b in pending:
                    work.wait()
                    if division:
                        flat.div_(len(ranks))
                    comm._unpack(flat, b)
        return _Callback()


def MultiProcessDataParallelCommunicator(ctx=None):
    """One process per device, as python/src/nnabla/communicator.pyx:592-646 describes it."""
    return Communicator(ctx)


def DataParallelCommunicator(ctx=None):
    raise NotImplementedError("single-process multi-device communication is not provided: run one process per GPU "
                              "(MultiProcessDataParallelCommunicator)")
