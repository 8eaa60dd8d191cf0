"""Host-side multi-rank logic on CPU: world_size-2 gloo process group (no GPU)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from torch_points_kernels_b200 import sharding


def test_shard_range_covers_everything():
    for n in (0, 1, 7, 16, 33):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_balanced_blocks():
    costs = [5, 1, 1, 1, 8, 2, 2, 4]
    b = sharding.balanced_blocks(costs, 3)
    assert b[0] == 0 and b[-1] == len(costs) and len(b) == 4 and b == sorted(b)
    loads = [sum(costs[b[i]:b[i + 1]]) for i in range(3)]
    assert max(loads) <= 1.5 * sum(costs) / 3
    assert sharding.balanced_blocks([1, 1], 4)[-1] == 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        d1 = torch.rand(6, 50, generator=g)   # what the 6 pairs' dist1 / dist2 would be
        d2 = torch.rand(6, 70, generator=g)
        lo, hi = sharding.shard_range(6, rank, world)
        loss = sharding.reduce_chamfer_loss(d1[lo:hi].sum(), d1[lo:hi].numel(), d2[lo:hi].sum(), d2[lo:hi].numel())
        want = d1.mean() + d2.mean()
        out.put((rank, float(loss), float(want)))
    finally:
        dist.destroy_process_group()


def _worker_backward(rank, world, port, out):
    """Loss and gradients of the sharded chamfer reduction, per rank, against the
    single-process mean over the whole batch; plus the final gather of per-rank outputs
    (5 items over 2 ranks: uneven blocks)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(6)
        d1 = torch.rand(5, 40, generator=g)
        d2 = torch.rand(5, 30, generator=g)
        # single-process reference: loss and gradient of mean + mean w.r.t. every entry
        r1, r2 = d1.clone().requires_grad_(True), d2.clone().requires_grad_(True)
        ((r1 * r1).mean() + (r2 * r2).mean()).backward()
        lo, hi = sharding.shard_range(5, rank, world)
        a, b = d1[lo:hi].clone().requires_grad_(True), d2[lo:hi].clone().requires_grad_(True)
        loss = sharding.reduce_chamfer_loss((a * a).sum(), a.numel(), (b * b).sum(), b.numel())
        loss.backward()
        want = float((d1 * d1).mean() + (d2 * d2).mean())
        gathered = sharding.gather_outputs(d1[lo:hi], n_items=5)
        out.put((rank, abs(float(loss) - want), float((a.grad - r1.grad[lo:hi]).abs().max()),
                 float((b.grad - r2.grad[lo:hi]).abs().max()), bool(torch.equal(gathered, d1))))
    finally:
        dist.destroy_process_group()


def test_chamfer_loss_backward_and_final_gather_two_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_backward, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, dloss, dg1, dg2, same in results:
        assert dloss < 1e-6 and dg1 < 1e-8 and dg2 < 1e-8 and same


def test_chamfer_loss_reduction_two_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, got, want in results:
        assert abs(got - want) < 1e-6


def test_single_process_reduction_is_a_plain_mean():
    d1, d2 = torch.rand(3, 10), torch.rand(3, 20)
    got = sharding.reduce_chamfer_loss(d1.sum(), d1.numel(), d2.sum(), d2.numel())
    assert abs(float(got) - float(d1.mean() + d2.mean())) < 1e-6


def _worker_ragged(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # a packed batch of 5 segments; ranks take blocks balanced by points x queries
        nx, ny = [40, 10, 10, 10, 30], [4, 1, 1, 1, 3]
        bx = torch.cat([torch.full((n,), i, dtype=torch.int64) for i, n in enumerate(nx)])
        by = torch.cat([torch.full((n,), i, dtype=torch.int64) for i, n in enumerate(ny)])
        s0, s1, px0, px1, py0, py1 = sharding.packed_block(bx, by, rank, world)
        rows = torch.arange(py0, py1, dtype=torch.int64).view(-1, 1) * 10 + rank   # this rank's per-query result
        whole = sharding.gather_ragged(rows)
        out.put((rank, (s0, s1, px0, px1, py0, py1), whole[:, 0].tolist()))
    finally:
        dist.destroy_process_group()


def test_packed_blocks_and_ragged_gather_two_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_ragged, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, b0, w0), (_, b1, w1) = res
    # blocks are contiguous, cover all segments, points and queries, and are balanced by cost
    assert b0[0] == 0 and b0[1] == b1[0] and b1[1] == 5
    assert b0[2] == 0 and b0[3] == b1[2] and b1[3] == 100 and b0[4] == 0 and b0[5] == b1[4] and b1[5] == 10
    assert b0[1] == 1                         # cost 160 of 280 in the first segment
    # every rank holds every query's row, in query order; the last digit says which rank computed it
    assert w0 == w1 and [v // 10 for v in w0] == list(range(10))
    assert [v % 10 for v in w0] == [0] * 4 + [1] * 6
