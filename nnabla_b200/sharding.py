"""Sharding of the quantized-layer path over the GPUs of one box (one process per GPU).

* Elementwise quantizers: contiguous element slices, no collective.
* A single large affine: OUTPUT COLUMNS. Rank r owns W[:, c0:c1] (and for a
  binary-weight layer its own alpha[c0:c1], since alpha is per output column,
  src/nbla/function/generic/binary_weight_affine.cpp:92-98), every rank holds
  the full x; the only exchange is an all-gather of the [rows, c1-c0] output
  slabs, interleaved back into the row-major [rows, N] result.
* Convolutions and whole networks: the BATCH; weights replicated; no exchange
  during forward.

torch.distributed is the plumbing (NCCL on GPUs, gloo in the CPU tests).
"""
import torch
import torch.distributed as dist


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
