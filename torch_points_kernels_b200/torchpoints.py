"""Python/autograd surface of the sampling, search, interpolation and grouping ops.

Same names, argument order, defaults, return order, dtypes and exception types as
torch_points_kernels/torchpoints.py of the reference; every op runs a hand-written
sm_100a kernel through the C ABI in include/tpk_b200.h.  Tensors must live on a CUDA
device: there is no CPU path.
"""
from typing import Optional

import torch
from torch.autograd import Function

from . import _lib
from .knn import knn  # noqa: F401  (re-exported like the reference does)


def _f32(t, name):
    _lib.check_contiguous(t, name)
    _lib.check_float(t, name)
    _lib.check_cuda(t, name)
    # the reference kernels read float32 only (DATA_PTR<float>)
    if t.dtype != torch.float32:
        raise RuntimeError("%s must be a float32 tensor" % name)
    return t


def furthest_point_sample(xyz, npoint, return_xyz=False):
    r"""
    Iterative furthest point sampling (reference: torchpoints.py:14-37,
    cuda/src/sampling.cpp:8-25).

    Parameters
    ----------
    xyz : torch.Tensor
        (B, N, 3) float32 CUDA tensor where N >= npoint
    npoint : int
        number of points in the sampled set
    return_xyz : bool
        also return the coordinates of the samples, (B, npoint, 3): the same values as
        ``xyz.gather(1, idx.long()[..., None].expand(-1, -1, 3))``, gathered by one small kernel
        behind the sampling kernel (an addition to the reference's signature)

    Returns
    -------
    torch.Tensor
        (B, npoint) int32 tensor of indices; the first one is always 0
        (with ``return_xyz``: the tuple (indices, coordinates))
    """
    if npoint > xyz.shape[1]:
        raise ValueError("caanot sample %i points from an input set of %i points" % (npoint, xyz.shape[1]))
    _f32(xyz, "points")
    b, n = xyz.shape[0], xyz.shape[1]
    out = torch.empty((b, npoint), dtype=torch.int32, device=xyz.device)
    new_xyz = torch.empty((b, npoint, 3), dtype=torch.float32, device=xyz.device) if return_xyz else None
    scratch = None
    with torch.cuda.device(xyz.device):
        need = _lib.lib().tpk_fps_scratch_bytes(b, n, npoint)
        if need < 0:
            raise RuntimeError("furthest_point_sample: clouds of %d points are not supported" % n)
        if need > 0:
            scratch = torch.empty((need,), dtype=torch.uint8, device=xyz.device)
        _lib.call("tpk_furthest_point_sampling_xyz", b, n, npoint, _lib.ptr(xyz), _lib.ptr(scratch),
                  max(need, 0), _lib.ptr(out), _lib.ptr(new_xyz), _lib.stream_of(xyz))
    return (out, new_xyz) if return_xyz else out


def three_nn(unknown, known):
    r"""
    Three nearest neighbours of ``unknown`` in ``known`` (reference: torchpoints.py:40-64).

    Parameters
    ----------
    unknown : torch.Tensor
        (B, n, 3) float32 CUDA tensor
    known : torch.Tensor
        (B, m, 3) float32 CUDA tensor

    Returns
    -------
    dist : torch.Tensor
        (B, n, 3) l2 distance to the three nearest neighbours
    idx : torch.Tensor
        (B, n, 3) int32 index of the three nearest neighbours
    """
    if unknown.shape[1] < 3:
        raise ValueError("Not enough points. unknown should ahve at least 3 points.")
    _f32(unknown, "unknowns")
    _f32(known, "knows")
    b, n = unknown.shape[0], unknown.shape[1]
    m = known.shape[1]
    dist2 = torch.empty((b, n, 3), dtype=torch.float32, device=unknown.device)
    idx = torch.empty((b, n, 3), dtype=torch.int32, device=unknown.device)
    with torch.cuda.device(unknown.device):
        need = _lib.lib().tpk_three_nn_scratch_bytes(b, n, m)
        if need > 0:
            # many known points: uniform-grid search with scratch (same results as the scan)
            scratch = torch.empty((need,), dtype=torch.uint8, device=unknown.device)
            _lib.call("tpk_three_nn_ws", b, n, m, _lib.ptr(unknown), _lib.ptr(known), _lib.ptr(dist2),
                      _lib.ptr(idx), _lib.ptr(scratch), need, _lib.stream_of(unknown))
        else:
            _lib.call("tpk_three_nn", b, n, m, _lib.ptr(unknown), _lib.ptr(known), _lib.ptr(dist2),
                      _lib.ptr(idx), _lib.stream_of(unknown))
    return torch.sqrt(dist2), idx


def three_interpolate_backward(grad_out, idx, weight, m):
    """Gradient of three_interpolate w.r.t. its features: (B, c, n) -> (B, c, m), the scatter-add
    of grad_out * weight (reference: cuda/src/interpolate_gpu.cu:122-152).  What
    ThreeInterpolate.backward runs; callable on its own."""
    grad_out = grad_out.contiguous()
    _f32(grad_out, "grad_out")
    B, c, n = grad_out.size()
    grad_features = torch.empty((B, c, m), dtype=torch.float32, device=grad_out.device)
    with torch.cuda.device(grad_out.device):
        _lib.call("tpk_three_interpolate_grad", B, c, n, m, _lib.ptr(grad_out), _lib.ptr(idx),
                  _lib.ptr(weight), _lib.ptr(grad_features), _lib.stream_of(grad_out))
    return grad_features


class ThreeInterpolate(Function):
    """Weighted sum of three gathered feature columns (reference: torchpoints.py:67-106)."""

    @staticmethod
    def forward(ctx, features, idx, weight):
        B, c, m = features.size()
        n = idx.size(1)
        ctx.three_interpolate_for_backward = (idx, weight, m)
        _f32(features, "points")
        _lib.check_contiguous(idx, "idx")
        _lib.check_int(idx, "idx")
        _lib.check_cuda(idx, "idx")
        _f32(weight, "weight")
        if idx.dtype != torch.int32:
            raise RuntimeError("idx must be an int32 tensor")
        out = torch.empty((B, c, n), dtype=torch.float32, device=features.device)
        with torch.cuda.device(features.device):
            _lib.call("tpk_three_interpolate", B, c, m, n, _lib.ptr(features), _lib.ptr(idx),
                      _lib.ptr(weight), _lib.ptr(out), _lib.stream_of(features))
            if _lib.debug_checks():
                _lib.raise_on_device_status("three_interpolate")
        return out

    @staticmethod
    def backward(ctx, grad_out):
        idx, weight, m = ctx.three_interpolate_for_backward
        return three_interpolate_backward(grad_out, idx, weight, m), None, None


def three_interpolate(features, idx, weight):
    r"""
    Weighted linear interpolation from three neighbours (reference: torchpoints.py:109-126).

    Parameters
    ----------
    features : torch.Tensor
        (B, c, m) features to interpolate from
    idx : torch.Tensor
        (B, n, 3) int32 three nearest neighbours of the target points in features
    weight : torch.Tensor
        (B, n, 3) weights

    Returns
    -------
    torch.Tensor
        (B, c, n) tensor of the interpolated features
    """
    return ThreeInterpolate.apply(features, idx, weight)


def grouping_backward(grad_out, idx, n):
    """Gradient of grouping_operation w.r.t. its features: (B, c, npoint, nsample) -> (B, c, n),
    the scatter-add autograd derives for the reference's torch.gather
    (torch_points_kernels/torchpoints.py:143-146).  What GroupingOperation.backward runs."""
    grad_out = grad_out.contiguous()
    _f32(grad_out, "grad_out")
    B, c, npoint, nsample = grad_out.size()
    grad_features = torch.empty((B, c, n), dtype=torch.float32, device=grad_out.device)
    with torch.cuda.device(grad_out.device):
        # scratch for the inverted index (positions sorted by target); 0 bytes = shapes the sorted
        # kernels do not cover, which take the atomic kernels
        need = _lib.lib().tpk_grouping_grad_scratch_bytes(B, c, n, npoint, nsample)
        scratch = torch.empty(need, dtype=torch.uint8, device=grad_out.device) if need > 0 else None
        _lib.call("tpk_grouping_grad_ws", B, c, n, npoint, nsample, _lib.ptr(grad_out),
                  _lib.ptr(idx), _lib.ptr(grad_features), _lib.ptr(scratch) if scratch is not None else None,
                  need, _lib.stream_of(grad_out))
    return grad_features


class GroupingOperation(Function):
    """Gather of feature columns by neighbourhood index; backward is a scatter-add."""

    @staticmethod
    def forward(ctx, features, idx):
        _f32(features, "features")
        _lib.check_contiguous(idx, "idx")
        _lib.check_cuda(idx, "idx")
        if idx.dtype != torch.int64:
            raise RuntimeError("gather(): Expected dtype int64 for index")
        B, c, n = features.size()
        _, npoint, nsample = idx.size()
        ctx.grouping_for_backward = (idx, n)
        out = torch.empty((B, c, npoint, nsample), dtype=torch.float32, device=features.device)
        with torch.cuda.device(features.device):
            _lib.call("tpk_grouping", B, c, n, npoint, nsample, _lib.ptr(features), _lib.ptr(idx),
                      _lib.ptr(out), _lib.stream_of(features))
            if _lib.debug_checks():
                _lib.raise_on_device_status("grouping_operation")
        return out

    @staticmethod
    def backward(ctx, grad_out):
        idx, n = ctx.grouping_for_backward
        return grouping_backward(grad_out, idx, n), None


def grouping_operation(features, idx):
    r"""
    Groups features by neighbourhood (reference: torchpoints.py:129-146, a torch.gather
    on an expanded index there; one gather kernel and one scatter-add kernel here).

    Parameters
    ----------
    features : torch.Tensor
        (B, C, N) tensor of features to group
    idx : torch.Tensor
        (B, npoint, nsample) int64 tensor containing the indicies of features to group with

    Returns
    -------
    torch.Tensor
        (B, C, npoint, nsample) tensor
    """
    return GroupingOperation.apply(features, idx)


class SAGroup(Function):
    """Fused grouping step of a set-abstraction layer (see sa_group)."""

    @staticmethod
    def forward(ctx, xyz, features, fps_idx, radius, nsample):
        _f32(xyz, "xyz")
        _lib.check_contiguous(fps_idx, "fps_idx")
        _lib.check_cuda(fps_idx, "fps_idx")
        if fps_idx.dtype != torch.int32:
            raise RuntimeError("fps_idx must be an int32 tensor (what furthest_point_sample returns)")
        b, n = xyz.shape[0], xyz.shape[1]
        m = fps_idx.shape[1]
        c = 0
        if features is not None:
            _f32(features, "features")
            c = features.shape[1]
        new_xyz = torch.empty((b, m, 3), dtype=torch.float32, device=xyz.device)
        idx = torch.empty((b, m, nsample), dtype=torch.int64, device=xyz.device)
        out = torch.empty((b, 3 + c, m, nsample), dtype=torch.float32, device=xyz.device)
        with torch.cuda.device(xyz.device):
            need = _lib.lib().tpk_sa_group_scratch_bytes(b, n, m, int(nsample))
            scratch = torch.empty((max(need, 1),), dtype=torch.uint8, device=xyz.device)
            _lib.call("tpk_sa_group", b, n, m, c, float(radius), int(nsample), _lib.ptr(xyz), _lib.ptr(features),
                      _lib.ptr(fps_idx), _lib.ptr(new_xyz), _lib.ptr(idx), _lib.ptr(out), _lib.ptr(scratch), need,
                      _lib.stream_of(xyz))
        ctx.sa_group_for_backward = (idx, n, c)
        ctx.mark_non_differentiable(new_xyz, idx)
        return new_xyz, idx, out

    @staticmethod
    def backward(ctx, _g_new_xyz, _g_idx, grad_out):
        idx, n, c = ctx.sa_group_for_backward
        grad_features = None
        if c > 0:
            # the feature rows of the gradient; the coordinates get none (indices and centres are
            # selections, and PointNet++ does not train through the point positions)
            # read in place (tpk_sa_group_grad takes the whole (B, 3+c, npoint, nsample) gradient)
            grad_out = grad_out.contiguous()
            _f32(grad_out, "grad_out")
            B, _, npoint, nsample = grad_out.size()
            grad_features = torch.empty((B, c, n), dtype=torch.float32, device=grad_out.device)
            with torch.cuda.device(grad_out.device):
                need = _lib.lib().tpk_grouping_grad_scratch_bytes(B, c, n, npoint, nsample)
                scratch = torch.empty(need, dtype=torch.uint8, device=grad_out.device) if need > 0 else None
                _lib.call("tpk_sa_group_grad", B, c, n, npoint, nsample, _lib.ptr(grad_out), _lib.ptr(idx),
                          _lib.ptr(grad_features), _lib.ptr(scratch), need, _lib.stream_of(grad_out))
        return None, grad_features, None, None, None


def sa_group(xyz, features, fps_idx, radius, nsample):
    r"""
    Grouping step of a PointNet++ set-abstraction layer as one fused call: the sequence
    ``new_xyz = gather(xyz, fps_idx)``; ``idx, _ = ball_query(radius, nsample, xyz, new_xyz)``;
    ``cat([grouping_operation(xyz^T, idx) - new_xyz^T[..., None], grouping_operation(features, idx)], 1)``
    of the reference's callers (torchpoints.py:129-146, 171-218), bit-identical to it, without
    materialising the intermediate tensors.  No counterpart in the reference.

    Parameters
    ----------
    xyz : torch.Tensor
        (B, N, 3) float32 CUDA tensor
    features : torch.Tensor or None
        (B, C, N) float32 features of the points
    fps_idx : torch.Tensor
        (B, M) int32 indices of the centres (what furthest_point_sample returns)
    radius, nsample :
        the ball query's parameters

    Returns
    -------
    new_xyz : (B, M, 3) centres
    idx : (B, M, nsample) int64 neighbour indices
    new_features : (B, 3 + C, M, nsample), relative coordinates first; differentiable w.r.t. features
    """
    return SAGroup.apply(xyz, features, fps_idx, radius, nsample)


def ball_query_dense(radius, nsample, xyz, new_xyz, batch_xyz=None, batch_new_xyz=None, sort=False):
    """Reference: torchpoints.py:149-157 -> cuda/src/ball_query.cpp:15-36."""
    if sort:
        raise NotImplementedError("CUDA version does not sort the neighbors")
    _f32(new_xyz, "new_xyz")
    _f32(xyz, "xyz")
    b, m = new_xyz.shape[0], new_xyz.shape[1]
    n = xyz.shape[1]
    idx = torch.empty((b, m, nsample), dtype=torch.int64, device=new_xyz.device)
    dist = torch.empty((b, m, nsample), dtype=torch.float32, device=new_xyz.device)
    with torch.cuda.device(new_xyz.device):
        need = _lib.lib().tpk_ball_query_dense_scratch_bytes(b, n, m, int(nsample))
        if need > 0:
            # large clouds: uniform-grid search with scratch (same results as the scan)
            scratch = torch.empty((need,), dtype=torch.uint8, device=new_xyz.device)
            _lib.call("tpk_ball_query_dense_ws", b, n, m, float(radius), int(nsample), _lib.ptr(new_xyz),
                      _lib.ptr(xyz), _lib.ptr(idx), _lib.ptr(dist), _lib.ptr(scratch), need,
                      _lib.stream_of(new_xyz))
        else:
            _lib.call("tpk_ball_query_dense", b, n, m, float(radius), int(nsample), _lib.ptr(new_xyz),
                      _lib.ptr(xyz), _lib.ptr(idx), _lib.ptr(dist), _lib.stream_of(new_xyz))
    return idx, dist


def ball_query_partial_dense(radius, nsample, x, y, batch_x, batch_y, sort=False):
    """Reference: torchpoints.py:160-168 -> cuda/src/ball_query.cpp:45-81."""
    if sort:
        raise NotImplementedError("CUDA version does not sort the neighbors")
    _f32(x, "x")
    _f32(y, "y")
    _lib.check_cuda(batch_x, "batch_x")
    _lib.check_cuda(batch_y, "batch_y")
    if batch_x.dtype != torch.int64 or batch_y.dtype != torch.int64:
        raise RuntimeError("batch_x and batch_y must be int64 tensors")
    batch_x = batch_x.contiguous()
    batch_y = batch_y.contiguous()
    if _lib.debug_checks():
        _lib.check_segments(batch_x, batch_y)
    ny = y.shape[0]
    idx = torch.empty((ny, nsample), dtype=torch.int64, device=y.device)
    dist = torch.empty((ny, nsample), dtype=torch.float32, device=y.device)
    with torch.cuda.device(y.device):
        need = _lib.lib().tpk_ball_query_partial_dense_scratch_bytes(x.shape[0], ny, float(radius))
        if need > 0:
            # hashed uniform grid with scratch (same results as the scan of the segments)
            scratch = torch.empty((need,), dtype=torch.uint8, device=y.device)
            _lib.call("tpk_ball_query_partial_dense_ws", x.shape[0], ny, float(radius), int(nsample),
                      _lib.ptr(x), _lib.ptr(y), _lib.ptr(batch_x), _lib.ptr(batch_y), _lib.ptr(idx),
                      _lib.ptr(dist), _lib.ptr(scratch), need, _lib.stream_of(y))
        else:
            _lib.call("tpk_ball_query_partial_dense", x.shape[0], ny, float(radius), int(nsample),
                      _lib.ptr(x), _lib.ptr(y), _lib.ptr(batch_x), _lib.ptr(batch_y), _lib.ptr(idx),
                      _lib.ptr(dist), _lib.stream_of(y))
    return idx, dist


def ball_query(
    radius: float,
    nsample: int,
    x: torch.Tensor,
    y: torch.Tensor,
    mode: Optional[str] = "dense",
    batch_x: Optional[torch.Tensor] = None,
    batch_y: Optional[torch.Tensor] = None,
    sort: Optional[bool] = False,
):
    """
    Radius search (reference: torchpoints.py:171-218).

    Arguments:
        radius {float} -- radius of the balls
        nsample {int} -- maximum number of features in the balls
        x {torch.Tensor} --
            (M, 3) [partial_dense] or (B, M, 3) [dense] xyz coordinates of the features
        y {torch.Tensor} --
            (npoint, 3) [partial_dense] or or (B, npoint, 3) [dense] centers of the ball query
        mode {str} -- switch between "dense" or "partial_dense" data layout

    Keyword Arguments:
        batch_x -- (M, ) [partial_dense] sorted int64 segment id of every feature point
        batch_y -- (npoint, ) [partial_dense] sorted int64 segment id of every centre
        sort -- not supported on CUDA (raises NotImplementedError, as the reference does)

    Returns:
        idx: (npoint, nsample) or (B, npoint, nsample) [dense] int64 indexes of the elements
             of x within radius of y
        dist: same shape, squared distances; unused slots hold -1
    """
    if mode is None:
        raise Exception('The mode should be defined within ["partial_dense | dense"]')

    if mode.lower() == "partial_dense":
        if (batch_x is None) or (batch_y is None):
            raise Exception("batch_x and batch_y should be provided")
        assert x.size(0) == batch_x.size(0)
        assert y.size(0) == batch_y.size(0)
        assert x.dim() == 2
        return ball_query_partial_dense(radius, nsample, x, y, batch_x, batch_y, sort=sort)

    elif mode.lower() == "dense":
        if (batch_x is not None) or (batch_y is not None):
            raise Exception("batch_x and batch_y should not be provided")
        assert x.dim() == 3
        return ball_query_dense(radius, nsample, x, y, sort=sort)
    else:
        raise Exception("unrecognized mode {}".format(mode))
