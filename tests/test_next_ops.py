"""The ops either side of the spatial-search path: region growing, instance IoU, and the GRNet
ops gridding and cubic feature sampling.  CPU tests pin the oracle on the reference's own test
vectors; GPU tests compare the kernels with the oracle, with the reference's CUDA build where it
is present, and run the reference's float64 gradchecks."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import data

DEV = "cuda:0"
_REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _neighbour_lists(pos, batch, radius, nsample):
    """First nsample neighbours within radius (inclusive), same segment, index order, -1 padded:
    what the packed ball query returns (the oracle's version of it)."""
    idx, _ = orc.ball_query_partial(radius, nsample, pos, pos, batch, batch)
    return idx


def _iou_inputs(gt, batch, proposals):
    gt, batch = np.asarray(gt, np.int64), np.asarray(batch, np.int64)
    nsamples = int(batch[-1]) + 1
    num_gt = np.array([gt[batch == s].max() for s in range(nsamples)], np.int64)
    off = np.concatenate([[0], num_gt.cumsum()]).astype(np.int64)
    sizes = np.array([np.sum((gt == i) & (batch == s)) for s in range(nsamples) for i in range(1, num_gt[s] + 1)], np.int64)
    offsets = np.concatenate([[0], np.cumsum([len(p) for p in proposals])]).astype(np.int64)
    return num_gt, np.concatenate(proposals).astype(np.int64), offsets, gt, off, batch, sizes


# ------------------------------------------------------------------- oracle on CPU

def test_oracle_grow_proximity_known_answers(known_answers):
    ka = known_answers["grow_proximity"]
    pos, batch = np.asarray(ka["pos"], np.float32), np.asarray(ka["batch"], np.int64)
    nb = _neighbour_lists(pos, batch, ka["radius"], 16)
    assert orc.grow_proximity(nb, 1) == ka["clusters_min1"]
    assert orc.grow_proximity(nb, 3) == ka["clusters_min3"]


def test_oracle_instance_iou_known_answers(known_answers):
    for name in ("instance_iou_simple", "instance_iou_batch"):
        ka = known_answers[name]
        batch = ka.get("batch", [0] * len(ka["gt_instances"]))
        got = orc.instance_iou(*_iou_inputs(ka["gt_instances"], batch, ka["proposals"]))
        np.testing.assert_allclose(got, np.asarray(ka["iou"], np.float32), rtol=1e-4, atol=1e-6)


def test_oracle_gridding_conserves_mass_and_matches_finite_differences():
    g = data.gen(1)
    p = torch.rand(2, 50, 3, generator=g) * 6.8 - 3.9              # inside the grid [-4, 3]
    grid, w, ix = orc.gridding(p, 4)
    np.testing.assert_allclose(grid.sum(axis=1), 50.0, rtol=1e-5)  # trilinear weights of a point sum to one
    assert ix.min() >= 0 and ix.max() < 512
    gg = torch.randn(2, 512, generator=g).numpy()
    grad = orc.gridding_grad(w, ix, gg)
    eps = 1e-2
    q = p.clone()
    q[0, 7, 1] += eps
    fd = ((orc.gridding(q, 4)[0] - grid) * gg).sum() / eps
    assert abs(fd - grad[0, 7, 1]) < 5e-2 * max(1.0, abs(fd))


def test_oracle_cubic_feature_sampling_small_case():
    cf = np.arange(2 * 8, dtype=np.float32).reshape(1, 2, 2, 2, 2)
    p = np.array([[[0.5, 0.5, 0.5], [1.5, 0.2, 0.2]]], np.float32)
    out, ix = orc.cubic_feature_sampling(p, cf, 1)
    assert ix[0, 0].tolist() == list(range(8))
    np.testing.assert_array_equal(out[0, 0, :, 1], cf[0, 1].reshape(-1))
    assert ix[0, 1].tolist() == [4, 5, 6, 7, -1, -1, -1, -1] and (out[0, 1, 4:] == 0).all()
    back = orc.cubic_feature_sampling_grad(np.ones_like(out), ix, 2, 1)
    assert back.sum() == 2 * 12 and back[0, 0, 1, 0, 0] == 2


# ------------------------------------------------------------------------- GPU

@pytest.fixture(scope="module")
def ref_cuda():
    if not os.path.exists(os.path.join(_REF_DIR, "points_cuda.so")):
        return None
    sys.path.insert(0, _REF_DIR)
    try:
        import points_cuda
    except Exception:  # pragma: no cover - depends on the box
        return None
    return points_cuda


def _cu(t):
    return torch.as_tensor(t).to(DEV).contiguous()


@pytest.mark.gpu
def test_grow_proximity_and_region_grow_known_answers(known_answers):
    import torch_points_kernels_b200 as tpk

    ka = known_answers["grow_proximity"]
    pos, batch = _cu(np.asarray(ka["pos"], np.float32)), _cu(np.asarray(ka["batch"], np.int64))
    assert tpk.grow_proximity(pos, batch, radius=ka["radius"], min_cluster_size=1) == ka["clusters_min1"]
    assert tpk.grow_proximity(pos, batch, radius=ka["radius"], min_cluster_size=3) == ka["clusters_min3"]
    clusters = tpk.region_grow(pos, _cu(np.asarray(ka["labels"], np.int64)), batch, radius=ka["radius"], min_cluster_size=1)
    assert [c.tolist() for c in clusters] == known_answers["region_grow"]["clusters"]


@pytest.mark.gpu
@pytest.mark.parametrize("nsample,radius", [(16, 0.06), (4, 0.12), (48, 0.03)])
def test_grow_proximity_matches_sequential_traversal(nsample, radius):
    """Clusters of the label propagation against the reference's sequential traversal (oracle) on
    the same neighbour lists: small nsample truncates the lists, so the graph is directed."""
    import torch_points_kernels_b200 as tpk
    from torch_points_kernels_b200 import cluster

    x, _, bx, _ = data.packed_planes(n_scenes=3, lo=2000, hi=4000, seed=31)
    x = x / 5.0
    nb = tpk.ball_query(radius, nsample, _cu(x), _cu(x), mode="partial_dense", batch_x=_cu(bx), batch_y=_cu(bx))[0]
    want = orc.grow_proximity(nb.cpu().numpy(), 5)
    labels = cluster.cluster_labels(nb).cpu().numpy()
    # the label of a point is the seed (first member) of its cluster in the traversal
    seen = np.full(x.shape[0], -1, np.int64)
    for c in orc.grow_proximity(nb.cpu().numpy(), 1):
        seen[c] = c[0]
    np.testing.assert_array_equal(labels, seen)
    got = tpk.grow_proximity(_cu(x), _cu(bx), nsample=nsample, radius=radius, min_cluster_size=5)
    assert [sorted(c) for c in want] == got


@pytest.mark.gpu
def test_instance_iou_known_answers_and_reference(known_answers, ref_cuda):
    import torch_points_kernels_b200 as tpk

    for name in ("instance_iou_simple", "instance_iou_batch"):
        ka = known_answers[name]
        batch = _cu(np.asarray(ka["batch"], np.int64)) if "batch" in ka else None
        got = tpk.instance_iou([_cu(np.asarray(p, np.int64)) for p in ka["proposals"]],
                               _cu(np.asarray(ka["gt_instances"], np.int64)), batch=batch)
        np.testing.assert_allclose(got.cpu().numpy(), np.asarray(ka["iou"], np.float32), rtol=1e-4, atol=1e-6)
    # random batch: oracle bit for bit (same formula), reference CUDA kernel bit for bit
    g = data.gen(8)
    n = 5000
    batch = torch.sort(torch.randint(0, 4, (n,), generator=g)).values
    gt = torch.randint(0, 30, (n,), generator=g)
    proposals = []
    for s in range(4):
        pool = torch.nonzero(batch == s).flatten()
        for _ in range(10):
            k = int(torch.randint(5, 200, (1,), generator=g))
            proposals.append(pool[torch.randperm(pool.numel(), generator=g)[:k]])
    got = tpk.instance_iou([_cu(p) for p in proposals], _cu(gt), batch=_cu(batch)).cpu().numpy()
    args = _iou_inputs(gt.numpy(), batch.numpy(), [p.numpy() for p in proposals])
    np.testing.assert_array_equal(got.view(np.int32), orc.instance_iou(*args).view(np.int32))
    if ref_cuda is not None:
        num_gt, pidx, poff, gtl, off, b, sizes = (_cu(a) for a in args)
        want = ref_cuda.instance_iou_cuda(pidx, poff, gtl, sizes, num_gt, b)
        np.testing.assert_array_equal(got.view(np.int32), want.cpu().numpy().view(np.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("B,n,scale", [(2, 2048, 8), (1, 33, 4), (3, 5000, 32)])
def test_gridding_matches_oracle_and_reference(B, n, scale, ref_cuda):
    from torch_points_kernels_b200 import _lib
    from torch_points_kernels_b200.gridding import GriddingFunction

    g = data.gen(n)
    # strictly inside the grid [-scale, scale - 1]: the reference kernel has no bounds check
    p = (torch.rand(B, n, 3, generator=g) * (2 * scale - 1.02) - (scale - 0.01)).contiguous()
    p[0, 0] = torch.tensor([1.0, -2.0, 0.0])  # integer coordinates: upper = lower + 1
    x = _cu(p).requires_grad_(True)
    grid = GriddingFunction.apply(x, scale)
    og, ow, oi = orc.gridding(p, scale)
    np.testing.assert_allclose(grid.detach().cpu().numpy(), og, rtol=1e-5, atol=1e-5)
    gg = torch.randn(B, (2 * scale) ** 3, generator=g)
    grid.backward(_cu(gg))
    np.testing.assert_array_equal(x.grad.cpu().numpy().view(np.int32), orc.gridding_grad(ow, oi, gg).view(np.int32))
    assert _lib.device_status() == 0
    if ref_cuda is not None:
        s = float(scale)
        rg, rw, ri = ref_cuda.gridding(-s, s - 1, -s, s - 1, -s, s - 1, x.detach())
        torch.testing.assert_close(grid.detach(), rg, rtol=1e-5, atol=1e-5)
        np.testing.assert_array_equal(x.grad.cpu().numpy().view(np.int32),
                                      ref_cuda.gridding_grad(rw, ri, _cu(gg)).cpu().numpy().view(np.int32))


@pytest.mark.gpu
def test_gridding_wrapper_drops_padding_and_guards_the_grid():
    from torch_points_kernels_b200 import _lib, gridding

    g = data.gen(4)
    p = torch.rand(2, 100, 3, generator=g) * 1.7 - 0.9   # times 8: inside the grid [-8, 7]
    p[1, 50:] = 0  # padding: coordinates summing to zero are dropped
    out = gridding.gridding(_cu(p), 8)
    assert out.shape == (2, 16 ** 3)
    np.testing.assert_allclose(out.cpu().numpy().sum(axis=1), [100.0, 50.0], rtol=1e-4)
    # a point outside the grid contributes to the vertices that exist and to nothing else
    far = _cu(torch.tensor([[[7.5, 0.5, 0.5], [100.0, 0.0, 0.0]]]))
    grid = gridding.GriddingFunction.apply(far, 8)
    torch.cuda.synchronize()
    assert _lib.device_status() == 2
    np.testing.assert_allclose(float(grid.sum()), 0.5, rtol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("B,n,c,scale,ns", [(2, 1000, 16, 8, 1), (2, 500, 4, 8, 2), (1, 300, 2, 16, 3)])
def test_cubic_feature_sampling_matches_oracle_and_reference(B, n, c, scale, ns, ref_cuda):
    from torch_points_kernels_b200.cubic_feature_sampling import CubicFeatureSamplingFunction

    g = data.gen(n + ns)
    p = (torch.rand(B, n, 3, generator=g) * (scale + 2) - 1).contiguous()  # some points outside the grid
    cf = torch.randn(B, c, scale, scale, scale, generator=g)
    x, f = _cu(p), _cu(cf).requires_grad_(True)
    out = CubicFeatureSamplingFunction.apply(x, f, ns)
    oo, oi = orc.cubic_feature_sampling(p, cf, ns)
    np.testing.assert_array_equal(out.detach().cpu().numpy(), oo)
    gout = torch.randn(out.shape, generator=g)
    out.backward(_cu(gout))
    np.testing.assert_allclose(f.grad.cpu().numpy(), orc.cubic_feature_sampling_grad(gout, oi, scale, ns), rtol=1e-4, atol=1e-4)
    if ref_cuda is not None:
        ro, ri = ref_cuda.cubic_feature_sampling(scale, ns, x, f.detach())
        np.testing.assert_array_equal(out.detach().cpu().numpy(), ro.cpu().numpy())
        _, rgrad = ref_cuda.cubic_feature_sampling_grad(scale, ns, _cu(gout), ri)
        torch.testing.assert_close(f.grad, rgrad, rtol=1e-4, atol=1e-4)


@pytest.mark.gpu
def test_grnet_float64_gradchecks():
    """The reference's own tests: test/test_gridding.py:21-31, test/test_cubic_feature_sampling.py:20-55."""
    from torch.autograd import gradcheck

    from torch_points_kernels_b200.cubic_feature_sampling import CubicFeatureSamplingFunction
    from torch_points_kernels_b200.gridding import GriddingFunction

    g = data.gen(6)
    for n, scale in ((32, 4), (64, 8)):
        x = torch.rand(1, n, 3, generator=g).double().to(DEV).requires_grad_(True)
        assert gradcheck(GriddingFunction.apply, [x, scale])
    for shape, cshape, ns in (((2, 64, 3), (2, 4, 8, 8, 8), 1), ((2, 32, 3), (2, 2, 8, 8, 8), 2), ((1, 32, 3), (1, 2, 16, 16, 16), 3)):
        p = (torch.rand(*shape, generator=g) * 2 - 1).double().to(DEV).requires_grad_(True)
        cf = torch.rand(*cshape, generator=g).double().to(DEV).requires_grad_(True)
        assert gradcheck(CubicFeatureSamplingFunction.apply, [p, cf, ns])
