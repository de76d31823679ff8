"""Sharding of the quantized-layer path over the GPUs of one box (one process per GPU).

* Elementwise quantizers: contiguous element slices, no collective.
* A single large affine: OUTPUT COLUMNS. Rank r owns W[:, c0:c1] (and for a
  binary-weight layer its own alpha[c0:c1], since alpha is per output column,
  src/nbla/function/generic/binary_weight_affine.cpp:92-98), every rank holds
  the full x; the only exchange is the gather of the [rows, c1-c0] output
  slabs into the row-major [rows, N] result, either as an all-gather after the
  contraction (gather_columns) or fused into the contraction's epilogue, which
  stores each slab straight into every rank's result (PeerMatrices).
* Convolutions and whole networks: the BATCH; weights replicated; no exchange
  during forward.

torch.distributed is the plumbing (NCCL on GPUs, gloo in the CPU tests).
"""
import ctypes

import torch
import torch.distributed as dist


class PeerLost(RuntimeError):
    """A rank did not reach a step within the deadline; `.missing` lists the ranks."""

    def __init__(self, step, missing, waited_s):
        RuntimeError.__init__(self, "step %s: rank(s) %s did not arrive within %.1f s" % (step, missing, waited_s))
        self.step, self.missing = step, missing


class StepGuard:
    """Host-side check that every rank is about to take part in a step, made BEFORE anything is
    launched for it. The kernels and collectives of this package never wait on another rank on
    the device, so a lost rank can only make a later collective (the gather, the ordering
    all-reduce of PeerMatrices.fence) wait for its own timeout; the guard turns that into an
    immediate, named error on the host instead. Each rank publishes "rank r reached step s" in the
    job's key-value store (a torch.distributed Store: TCPStore, FileStore, ...) and reads the
    others' marks with a deadline. A rank that leaves does so between steps, with nothing in
    flight; the survivors learn of it here, before their next launch."""

    def __init__(self, store, rank, world, timeout_s=10.0, prefix="nb200/step"):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout_s, self.prefix = float(timeout_s), prefix

    def _key(self, step, rank):
        return "%s/%s/%d" % (self.prefix, step, rank)

    def arrive(self, step):
        """Marks this rank as present at `step` and waits until every rank is; raises PeerLost
        naming the ranks that are not there when the deadline passes."""
        import datetime
        import time
        self.store.set(self._key(step, self.rank), b"1")
        t0 = time.monotonic()
        missing = []
        for r in range(self.world):
            if r == self.rank:
                continue
            left = self.timeout_s - (time.monotonic() - t0)
            try:
                self.store.wait([self._key(step, r)], datetime.timedelta(seconds=max(left, 0.05)))
            except Exception:  # noqa: BLE001 - the store's wait signals its timeout with a RuntimeError / DistStoreError
                missing.append(r)
        if missing:
            raise PeerLost(step, missing, time.monotonic() - t0)


def shard_range(total, rank, world):
    """[begin, end) of shard `rank` when `total` units are split as evenly as
    possible (the first total % world shards get one more)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world: %d/%d" % (rank, world))
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def column_shard(weight, bias, rank, world):
    """Column slab of a [K, N] weight (and [N] bias) owned by `rank`."""
    c0, c1 = shard_range(weight.shape[1], rank, world)
    w = weight[:, c0:c1].contiguous()
    b = bias[c0:c1].contiguous() if bias is not None else None
    return w, b, (c0, c1)


def gather_columns(y_shard, n_total, group=None):
    """All-gather of output-column slabs: every rank passes its [rows, n_r]
    slab and receives the full row-major [rows, n_total] matrix. Slabs may be
    ragged (n_total not divisible by the world size)."""
    world = dist.get_world_size(group)
    rows = y_shard.shape[0]
    widths = [shard_range(n_total, r, world) for r in range(world)]
    wmax = max(e - b for b, e in widths)
    if y_shard.shape[1] != widths[dist.get_rank(group)][1] - widths[dist.get_rank(group)][0]:
        raise ValueError("slab width does not match this rank's column range")
    if y_shard.shape[1] != wmax:  # pad ragged slabs to a common width
        pad = y_shard.new_zeros((rows, wmax))
        pad[:, :y_shard.shape[1]] = y_shard
        y_shard = pad
    flat = y_shard.new_empty((world * rows, wmax))  # slabs concatenated along dim 0
    dist.all_gather_into_tensor(flat, y_shard.contiguous(), group=group)
    stage = flat.view(world, rows, wmax)
    out = y_shard.new_empty((rows, n_total))
    for r, (b, e) in enumerate(widths):
        out[:, b:e] = stage[r, :, :e - b]
    return out


def batch_shard(x, rank, world):
    b0, b1 = shard_range(x.shape[0], rank, world)
    return x[b0:b1]


def gather_batch(y_shard, n_total, group=None):
    """All-gather of batch shards (e.g. the logits of a batch-sharded network)."""
    world = dist.get_world_size(group)
    sizes = [shard_range(n_total, r, world) for r in range(world)]
    smax = max(e - b for b, e in sizes)
    tail = tuple(y_shard.shape[1:])
    buf = y_shard.new_zeros((smax,) + tail)
    buf[:y_shard.shape[0]] = y_shard
    flat = y_shard.new_empty((world * smax,) + tail)
    dist.all_gather_into_tensor(flat, buf, group=group)
    stage = flat.view((world, smax) + tail)
    return torch.cat([stage[r, :e - b] for r, (b, e) in enumerate(sizes)], 0)


class _DeviceArray:
    """A device allocation owned through the C ABI, exposed to torch via the CUDA array interface."""

    def __init__(self, addr, shape):
        self.addr = addr
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (addr, False),
                                         "version": 2, "strides": None}


class PeerMatrices:
    """One row-major [rows, cols] fp32 matrix per rank, each mapped into every
    rank's address space, for contractions that store their output-column slab
    into all ranks' results (functions.affine_from_codes_gather).

    Collective constructor: every rank of `group` allocates its matrix through
    the C ABI (nb200_malloc), exports it (nb200_ipc_export), the 64-byte
    handles are exchanged with all_gather_object, and each rank opens the
    others' (nb200_ipc_open). `ptrs[r]` is rank r's matrix as seen from this
    process, `local` a torch view of this rank's own matrix."""

    def __init__(self, rows, cols, group=None, device=None):
        from . import _capi as C
        self._C = C
        self.rows, self.cols, self.group = int(rows), int(cols), group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        nbytes = self.rows * self.cols * 4
        with torch.cuda.device(self.device):
            own = ctypes.c_void_p(0)
            C.call("nb200_malloc", ctypes.byref(own), C.size_t(nbytes))
            self._own = own.value
            handle = (ctypes.c_ubyte * 64)()
            C.call("nb200_ipc_export", ctypes.c_void_p(self._own), handle)
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            self.ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(self._own)
                    continue
                p = ctypes.c_void_p(0)
                C.call("nb200_ipc_open", (ctypes.c_ubyte * 64).from_buffer_copy(h), ctypes.byref(p))
                self.ptrs.append(p.value)
        self.local = torch.as_tensor(_DeviceArray(self._own, (self.rows, self.cols)), device=self.device)
        self._flag = torch.zeros(1, device=self.device)

    def fence(self):
        """Orders the ranks on the current stream: work enqueued after it sees
        every rank's stores that were enqueued before it."""
        dist.all_reduce(self._flag, group=self.group)

    def close(self):
        """Collective: unmaps the peers' matrices, then frees this rank's own."""
        if self._own is None:
            return
        C = self._C
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for r, p in enumerate(self.ptrs):
                if r != self.rank:
                    C.call("nb200_ipc_close", ctypes.c_void_p(p))
            dist.barrier(self.group)  # nobody frees while a peer still has the array mapped
            self.local = None
            C.call("nb200_free", ctypes.c_void_p(self._own))
        self._own, self.ptrs = None, []
