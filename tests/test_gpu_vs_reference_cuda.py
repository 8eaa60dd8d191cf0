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
