"""GPU tests against the reference's own CUDA extension, compiled for sm_100a from the
reference sources by oracle/Makefile (target ref_cuda) into oracle/_ref/points_cuda.so.
They pin what only the CUDA build defines: which products nvcc fused into FMAs (the
returned distances are compared bit for bit), the FPS tie order, index-order ball query.
Skipped when the extension has not been built."""
import os
import sys

import numpy as np
import pytest
import torch

import torch_points_kernels_b200 as tpk
from torch_points_kernels_b200 import chamfer_dist as cd
from tests import data

pytestmark = pytest.mark.gpu

_REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(os.path.join(_REF_DIR, "points_cuda.so")):
        pytest.skip("reference CUDA extension not built (make -C oracle ref_cuda)")
    sys.path.insert(0, _REF_DIR)
    try:
        import points_cuda
    except Exception as e:  # pragma: no cover - depends on the box
        pytest.skip("reference CUDA extension does not load here: %s" % e)
    return points_cuda


def eq_bits(a, b):
    np.testing.assert_array_equal(a.detach().cpu().numpy().view(np.int32), b.detach().cpu().numpy().view(np.int32))


def eq(a, b):
    np.testing.assert_array_equal(a.detach().cpu().numpy(), b.detach().cpu().numpy())


@pytest.mark.parametrize("B,N,m", [(4, 4096, 1024), (2, 16384, 512), (3, 300, 100), (2, 1000, 1000)])
def test_fps(ref, B, N, m):
    x = data.unit_ball(B, N, seed=N).cuda()
    eq(tpk.furthest_point_sample(x, m), ref.furthest_point_sampling(x, m))


def test_fps_lattice_ties(ref):
    g = data.gen(5)
    x = torch.randint(0, 4, (4, 2000, 3), generator=g).float().cuda()
    eq(tpk.furthest_point_sample(x, 64), ref.furthest_point_sampling(x, 64))


@pytest.mark.parametrize("r,ns", [(0.2, 32), (0.05, 8), (0.8, 32)])
def test_ball_query_dense(ref, r, ns):
    x, y, _ = data.cfg1_plumbing()
    x, y = x.cuda(), y.cuda()
    idx, dist = tpk.ball_query(r, ns, x, y, mode="dense")
    ridx, rdist = ref.ball_query_dense(y, x, r, ns)
    eq(idx, ridx)
    eq_bits(dist, rdist)


def test_ball_query_partial(ref):
    x, y, bx, by = data.packed_planes(n_scenes=6, lo=2000, hi=8000, seed=3003)
    x, y, bx, by = x.cuda(), y.cuda(), bx.cuda(), by.cuda()
    idx, dist = tpk.ball_query(0.05, 64, x, y, mode="partial_dense", batch_x=bx, batch_y=by)
    ridx, rdist = ref.ball_query_partial_dense(x, y, bx, by, 0.05, 64)
    eq(idx, ridx)
    eq_bits(dist, rdist)


def test_three_nn_and_interpolate(ref):
    g = data.gen(9)
    known = torch.rand(4, 1024, 3, generator=g).cuda()
    unknown = torch.rand(4, 4096, 3, generator=g).cuda()
    feat = torch.randn(4, 64, 1024, generator=g).cuda()
    dist, idx = tpk.three_nn(unknown, known)
    rd2, ridx = ref.three_nn(unknown, known)
    eq(idx, ridx)
    eq_bits(dist, torch.sqrt(rd2))
    w = 1.0 / (dist + 1e-8)
    w = (w / w.sum(2, keepdim=True)).contiguous()
    eq_bits(tpk.three_interpolate(feat, idx, w), ref.three_interpolate(feat, ridx, w))
    gout = torch.randn(4, 64, 4096, generator=g).cuda()
    f = feat.clone().requires_grad_(True)
    tpk.three_interpolate(f, idx, w).backward(gout)
    torch.testing.assert_close(f.grad, ref.three_interpolate_grad(gout, ridx, w, 1024), rtol=1e-4, atol=1e-4)


def test_chamfer(ref):
    c1, c2 = data.chamfer_pair(4, 2048, seed=4001)
    c1, c2 = c1.cuda().requires_grad_(True), c2.cuda().requires_grad_(True)
    d1, d2 = cd.ChamferFunction.apply(c1, c2)
    r1, r2, i1, i2 = ref.chamfer_dist(c1.detach(), c2.detach())
    eq_bits(d1, r1)
    eq_bits(d2, r2)
    g1, g2 = torch.randn_like(d1), torch.randn_like(d2)
    torch.autograd.backward([d1, d2], [g1, g2])
    rg1, rg2 = ref.chamfer_dist_grad(c1.detach(), c2.detach(), i1, i2, g1, g2)
    torch.testing.assert_close(c1.grad, rg1, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(c2.grad, rg2, rtol=1e-4, atol=1e-4)


# ------------------------------------------------------------- the configurations at full size
#
# The shapes the benchmark numbers are quoted on, compared with the reference's own CUDA
# kernels (and its CPU kd-tree for kNN, which has no CUDA counterpart) on the same inputs.

def _ref_cpu():
    if not os.path.exists(os.path.join(_REF_DIR, "points_cpu.so")):
        pytest.skip("reference CPU extension not built (make -C oracle ref_cpu)")
    sys.path.insert(0, _REF_DIR)
    try:
        import points_cpu
    except Exception as e:  # pragma: no cover - depends on the box
        pytest.skip("reference CPU extension does not load here: %s" % e)
    return points_cpu


@pytest.mark.parametrize("family", [None, "fps_unsorted"])
def test_full_size_sa_fp_stack(ref, family, monkeypatch):
    """Configuration 2, B=16 x N=16384, the whole chained stack: FPS to 4096/1024/256/64 (all
    4095/1023/255/63 rounds), ball query, grouping forward and backward, three_nn and
    three_interpolate forward and backward, every level on the outputs of the level before."""
    import bench

    data.use_paths(monkeypatch, family)
    xyz_h, sa_h, fp_h = bench.make_inputs(bench.B_CLOUDS, bench.N_POINTS, 2000)
    g = torch.Generator(device="cuda").manual_seed(77)
    pts = xyz_h.cuda()
    ns = bench.LEVELS["nsample"]
    for l, (m, r, c) in enumerate(zip(bench.LEVELS["npoint"], bench.LEVELS["radius"], bench.LEVELS["channels"])):
        idx, centres = tpk.furthest_point_sample(pts, m, return_xyz=True)
        eq(idx, ref.furthest_point_sampling(pts, m))
        eq_bits(centres, torch.gather(pts, 1, idx.long().unsqueeze(-1).expand(-1, -1, 3)))
        nbr, dist = tpk.ball_query(r, ns, pts, centres, mode="dense")
        rnbr, rdist = ref.ball_query_dense(centres, pts, r, ns)
        eq(nbr, rnbr)
        eq_bits(dist, rdist)
        # grouping: the reference is torch.gather on the expanded index and its autograd
        f = sa_h[l].cuda().requires_grad_(True)
        grouped = tpk.grouping_operation(f, nbr)
        fr = sa_h[l].cuda().requires_grad_(True)
        all_idx = rnbr.reshape(rnbr.shape[0], -1).unsqueeze(1).expand(-1, c, -1)
        want = fr.gather(2, all_idx).reshape(grouped.shape)
        eq_bits(grouped, want)
        gout = torch.randn(grouped.shape, device="cuda", generator=g)
        grouped.backward(gout)
        want.backward(gout)
        torch.testing.assert_close(f.grad, fr.grad, rtol=1e-4, atol=1e-4)
        del grouped, want, gout, all_idx, f, fr
        # feature propagation of the level: from its centres back to its input points
        d3, i3 = tpk.three_nn(pts, centres)
        rd2, ri3 = ref.three_nn(pts, centres)
        eq(i3, ri3)
        eq_bits(d3, torch.sqrt(rd2))
        w = 1.0 / (d3 + 1e-8)
        w = (w / w.sum(2, keepdim=True)).contiguous()
        ff = fp_h[l].cuda().requires_grad_(True)
        up = tpk.three_interpolate(ff, i3, w)
        eq_bits(up, ref.three_interpolate(ff.detach(), ri3, w))
        gup = torch.randn(up.shape, device="cuda", generator=g)
        up.backward(gup)
        torch.testing.assert_close(ff.grad, ref.three_interpolate_grad(gup, ri3, w, m), rtol=1e-4, atol=1e-4)
        pts = centres
    from torch_points_kernels_b200 import _lib
    assert _lib.device_status() == 0


def test_full_size_chamfer(ref):
    """Configuration 4: B=32 pairs of 16384 points, distances bit for bit, indices, gradients."""
    c1, c2 = data.chamfer_pair(32, 16384, seed=4000)
    x1, x2 = c1.cuda().requires_grad_(True), c2.cuda().requires_grad_(True)
    d1, d2 = cd.ChamferFunction.apply(x1, x2)
    r1, r2, i1, i2 = ref.chamfer_dist(x1.detach(), x2.detach())
    eq_bits(d1, r1)
    eq_bits(d2, r2)
    # the nearest neighbours themselves, through the C ABI
    from torch_points_kernels_b200 import _lib
    o1, o2 = torch.empty_like(r1), torch.empty_like(r2)
    j1, j2 = torch.empty_like(i1), torch.empty_like(i2)
    need = _lib.lib().tpk_chamfer_dist_scratch_bytes(32, 16384, 16384)
    scratch = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    _lib.call("tpk_chamfer_dist_f32_ws", 32, 16384, _lib.ptr(x1), 16384, _lib.ptr(x2), _lib.ptr(o1), _lib.ptr(o2),
              _lib.ptr(j1), _lib.ptr(j2), _lib.ptr(scratch), need, _lib.stream_of(x1))
    eq(j1, i1)
    eq(j2, i2)
    g1, g2 = torch.randn_like(d1), torch.randn_like(d2)
    torch.autograd.backward([d1, d2], [g1, g2])
    rg1, rg2 = ref.chamfer_dist_grad(x1.detach(), x2.detach(), i1, i2, g1, g2)
    torch.testing.assert_close(x1.grad, rg1, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(x2.grad, rg2, rtol=1e-4, atol=1e-4)


@pytest.fixture(scope="module")
def packed_scenes():
    return data.packed_planes(seed=3000)


def test_full_size_packed_ball_query(ref, packed_scenes):
    """Configuration 3: all 64 scenes (about 7 million points, 0.7 million queries) through the
    packed radius search, indices and distances bit for bit."""
    x, y, bx, by = (t.cuda() for t in packed_scenes)
    idx, dist = tpk.ball_query(0.05, 64, x, y, mode="partial_dense", batch_x=bx, batch_y=by)
    ridx, rdist = ref.ball_query_partial_dense(x, y, bx, by, 0.05, 64)
    eq(idx, ridx)
    eq_bits(dist, rdist)


def test_full_size_packed_knn(packed_scenes):
    """Configuration 3, kNN k=16 on the whole packed batch; four whole scenes are compared with
    the reference's kd-tree search run per scene (it has no packed kNN), indices offset by the
    scene's first point; every scene is checked for sorted distances and in-segment indices."""
    tpcpu = _ref_cpu()
    x, y, bx, by = packed_scenes
    idx, d2 = tpk.knn(x.cuda(), y.cuda(), 16, batch_support=bx.cuda(), batch_pos=by.cuda())
    idx, d2 = idx.cpu(), d2.cpu()
    offx = torch.searchsorted(bx, torch.arange(65))
    offy = torch.searchsorted(by, torch.arange(65))
    assert bool((d2[:, 1:] >= d2[:, :-1]).all())
    seg_lo, seg_hi = offx[by], offx[by + 1]
    assert bool(((idx >= seg_lo[:, None]) & (idx < seg_hi[:, None])).all())
    for s in (0, 17, 40, 63):
        xs = x[offx[s]:offx[s + 1]].unsqueeze(0).contiguous()
        ys = y[offy[s]:offy[s + 1]].unsqueeze(0).contiguous()
        ridx, rd2 = tpcpu.dense_knn(xs, ys, 16)
        np.testing.assert_array_equal(idx[offy[s]:offy[s + 1]].numpy(), ridx[0].numpy() + int(offx[s]))
        np.testing.assert_array_equal(d2[offy[s]:offy[s + 1]].numpy().view(np.int32), rd2[0].numpy().view(np.int32))


def test_full_size_large_cloud(ref):
    """Configuration 5, one cloud of 2^20 points: FPS to 2048 samples against the reference
    CUDA kernel, then the dense ball query (radius 0.02, nsample 32) around the samples against
    the reference CUDA kernel, and against the CPU oracle on a subset of 1000 centres."""
    from oracle import oracle as orc

    x = data.gaussian_mixture(1, 1 << 20, seed=5000).cuda()
    idx, centres = tpk.furthest_point_sample(x, 2048, return_xyz=True)
    eq(idx, ref.furthest_point_sampling(x, 2048))
    nbr, dist = tpk.ball_query(0.02, 32, x, centres, mode="dense")
    rnbr, rdist = ref.ball_query_dense(centres, x, 0.02, 32)
    eq(nbr, rnbr)
    eq_bits(dist, rdist)
    sub = centres[:, ::2][:, :1000].contiguous()
    oi, od = orc.ball_query_dense(0.02, 32, x.cpu(), sub.cpu())
    np.testing.assert_array_equal(nbr[:, ::2][:, :1000].cpu().numpy(), oi)
    np.testing.assert_array_equal(dist[:, ::2][:, :1000].cpu().numpy().view(np.int32), od.view(np.int32))
