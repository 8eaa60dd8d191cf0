"""Batch sharding of the path across the GPUs of one node.

Every op on the path is independent per cloud (dense layout), per segment (packed
layout) or per pair (chamfer), so ranks take contiguous blocks of clouds and no kernel
needs a collective.  The only exchange is the scalar chamfer loss: two partial sums and
two counts per rank, all-reduced with torch.distributed (NCCL on GPUs, gloo in the CPU
tests); `gather_outputs` assembles per-rank results on every rank where a caller wants the
whole batch.  The reference has no multi-device code at all.
"""
import torch
import torch.distributed as dist


def shard_range(n_items, rank, world_size):
    """[lo, hi) of the contiguous block of items rank owns; blocks differ by at most one."""
    base, extra = divmod(int(n_items), int(world_size))
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def balanced_blocks(costs, world_size):
    """Contiguous partition of segments into world_size blocks with near-equal total cost
    (cost of a packed segment = support points x query points for the brute-force search).
    Returns world_size + 1 boundaries.  Greedy on the prefix sum."""
    costs = [float(c) for c in costs]
    total = sum(costs)
    bounds = [0]
    acc = 0.0
    for i, c in enumerate(costs):
        remaining_blocks = world_size - len(bounds)
        if remaining_blocks == 0:
            break
        target = total * len(bounds) / world_size
        # close the block before item i if that lands nearer the target than after it
        if acc > 0 and abs(acc - target) <= abs(acc + c - target) and len(costs) - i >= remaining_blocks:
            bounds.append(i)
        acc += c
    while len(bounds) < world_size:
        bounds.append(len(costs))
    bounds.append(len(costs))
    return bounds


class _AllReduceSum(torch.autograd.Function):
    """Sum over the ranks of `group`.  Every rank ends up with the same value and calls
    backward on its own copy, so the gradient of that copy w.r.t. this rank's addend is the
    incoming gradient itself (no second collective)."""

    @staticmethod
    def forward(ctx, t, group):
        out = t.clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad, None


def reduce_chamfer_loss(sum1, count1, sum2, count2, group=None):
    """mean(dist1) + mean(dist2) over the clouds of ALL ranks from per-rank partial sums.

    sum1/sum2: 0-dim tensors (sum of this rank's dist1 / dist2 entries), count1/count2:
    number of entries behind them.  Matches the reference's single-device
    ``torch.mean(dist1) + torch.mean(dist2)`` (chamfer_dist.py:54) on the concatenated batch,
    and so do the gradients: backward() on the returned loss gives every rank the gradient
    of the whole batch's loss w.r.t. its own pairs.
    """
    buf = torch.stack([sum1.double(), sum2.double(),
                       torch.as_tensor(float(count1), dtype=torch.float64, device=sum1.device),
                       torch.as_tensor(float(count2), dtype=torch.float64, device=sum1.device)])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        buf = _AllReduceSum.apply(buf, group)
    return (buf[0] / buf[2] + buf[1] / buf[3]).to(sum1.dtype)


def chamfer_dist_sharded(xyz1, xyz2, group=None):
    """Chamfer loss of a batch whose pairs are spread over the ranks of `group`: every
    rank passes its own pairs, all ranks get the loss of the whole batch."""
    from .chamfer_dist import ChamferFunction

    dist1, dist2 = ChamferFunction.apply(xyz1, xyz2)
    return reduce_chamfer_loss(dist1.sum(), dist1.numel(), dist2.sum(), dist2.numel(), group)


def gather_outputs(t, n_items=None, group=None):
    """The "final gather": per-rank outputs (first dimension = this rank's items, blocks as
    shard_range hands them out) assembled into the whole batch's tensor on every rank with one
    all_gather_into_tensor.  Ranks whose block is one item shorter are padded for the
    collective and trimmed afterwards.  n_items: items of the whole batch (default: the
    blocks are equal, world_size x this rank's)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return t
    world = dist.get_world_size(group)
    if n_items is None:
        n_items = t.shape[0] * world
    per = -(-int(n_items) // world)
    send = t.contiguous()
    if send.shape[0] < per:
        pad = torch.zeros((per - send.shape[0],) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        send = torch.cat([send, pad])
    out = torch.empty((world * per,) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_gather_into_tensor(out, send, group=group)
    if per * world == n_items:
        return out
    parts = []
    for r in range(world):
        lo, hi = shard_range(n_items, r, world)
        parts.append(out[r * per:r * per + (hi - lo)])
    return torch.cat(parts)


def gather_ragged(t, group=None):
    """Per-rank outputs whose first dimension differs between ranks (the queries of a block of
    packed segments) assembled in rank order on every rank: the lengths travel in one small
    all_gather, the rows in one all_gather_into_tensor padded to the longest block."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return t
    world = dist.get_world_size(group)
    send = t.contiguous()
    mine = torch.tensor([send.shape[0]], dtype=torch.int64, device=send.device)
    lens = torch.empty(world, dtype=torch.int64, device=send.device)
    dist.all_gather_into_tensor(lens, mine, group=group)
    lens = [int(v) for v in lens.tolist()]
    per = max(lens)
    if send.shape[0] < per:
        pad = torch.zeros((per - send.shape[0],) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        send = torch.cat([send, pad])
    out = torch.empty((world * per,) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_gather_into_tensor(out, send, group=group)
    return torch.cat([out[r * per:r * per + lens[r]] for r in range(world)])


def packed_block(batch_x, batch_y, rank, world_size):
    """The contiguous block of segments rank takes from a packed batch, balanced by the cost of the
    brute-force search (support points x queries per segment).  batch_x / batch_y: sorted int64
    segment ids (host or device).  Returns (first segment, one past the last segment, first and
    one-past-last support point, first and one-past-last query)."""
    nseg = int(max(int(batch_x[-1]) if batch_x.numel() else -1, int(batch_y[-1]) if batch_y.numel() else -1)) + 1
    nx = torch.bincount(batch_x.cpu(), minlength=nseg)
    ny = torch.bincount(batch_y.cpu(), minlength=nseg)
    bounds = balanced_blocks((nx.double() * ny.double()).tolist(), world_size)
    s0, s1 = bounds[rank], bounds[rank + 1]
    cx = torch.cat([torch.zeros(1, dtype=torch.int64), nx.cumsum(0)])
    cy = torch.cat([torch.zeros(1, dtype=torch.int64), ny.cumsum(0)])
    return s0, s1, int(cx[s0]), int(cx[s1]), int(cy[s0]), int(cy[s1])
