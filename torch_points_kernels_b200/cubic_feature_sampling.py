"""Cubic feature sampling: features of the grid vertices around every point (reference:
torch_points_kernels/cubic_feature_sampling.py, kernels cuda/src/cubic_feature_sampling_gpu.cu)."""
import torch

from . import _lib
from .gridding import _suffix


class CubicFeatureSamplingFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ptcloud, cubic_features, neighborhood_size=1):
        sfx = _suffix(ptcloud, "ptcloud")
        if cubic_features.dtype != ptcloud.dtype:
            raise RuntimeError("ptcloud and cubic_features must have the same dtype")
        _lib.check_cuda(cubic_features, "cubic_features")
        ptcloud = ptcloud.contiguous()
        cubic_features = cubic_features.contiguous()
        scale = cubic_features.size(2)
        b, n = ptcloud.shape[0], ptcloud.shape[1]
        c = cubic_features.shape[1]
        nvert = (2 * int(neighborhood_size)) ** 3
        point_features = torch.empty((b, n, nvert, c), dtype=ptcloud.dtype, device=ptcloud.device)
        indexes = torch.empty((b, n, nvert), dtype=torch.int32, device=ptcloud.device)
        with torch.cuda.device(ptcloud.device):
            _lib.call("tpk_cubic_feature_sampling_" + sfx, b, n, c, scale, int(neighborhood_size), _lib.ptr(ptcloud),
                      _lib.ptr(cubic_features), _lib.ptr(point_features), _lib.ptr(indexes), _lib.stream_of(ptcloud))
        ctx.cubic_for_backward = (scale, int(neighborhood_size), c)
        ctx.save_for_backward(indexes)
        return point_features

    @staticmethod
    def backward(ctx, grad_point_features):
        (indexes,) = ctx.saved_tensors
        scale, neighborhood_size, c = ctx.cubic_for_backward
        grad_point_features = grad_point_features.contiguous()
        sfx = _suffix(grad_point_features, "grad_point_features")
        b, n = indexes.shape[0], indexes.shape[1]
        dt, dev = grad_point_features.dtype, grad_point_features.device
        grad_ptcloud = torch.empty((b, n, 3), dtype=dt, device=dev)
        grad_cubic = torch.empty((b, c, scale, scale, scale), dtype=dt, device=dev)
        with torch.cuda.device(dev):
            _lib.call("tpk_cubic_feature_sampling_grad_" + sfx, b, n, c, scale, neighborhood_size,
                      _lib.ptr(grad_point_features), _lib.ptr(indexes), _lib.ptr(grad_ptcloud), _lib.ptr(grad_cubic),
                      _lib.stream_of(grad_point_features))
        return grad_ptcloud, grad_cubic, None


def cubic_feature_sampling(ptcloud, cubic_features, neighborhood_size=1):
    r"""
    Sample the features of points from 3D feature maps that the point lies in.
    Please refer to https://arxiv.org/pdf/2006.03761 for more information

    Parameters
    ----------
    ptcloud : torch.Tensor (dtype=torch.float32)
        (B, n_pts, 3) point clouds containing n_pts points
    cubic_features : torch.Tensor (dtype=torch.float32)
        (B, c, m, m, m) 3D feature maps of sizes m x m x m and c channels
    neighborhood_size : int
        The neighborhood cubes to sample.
        neighborhood_size = 1 means to sample the cube that point lies in.
        neighborhood_size = 2 means to sample surrouding cubes (step = 1) of
        the cube that point lies in.

    Returns
    -------
    dist: torch.Tensor
        (B, n_pts, n_vertices, c), where n_vertices = (neighborhood_size * 2)^3
    """
    if len(ptcloud.shape) != 3 or ptcloud.shape[2] != 3:
        raise ValueError("The input point cloud should be of size (B, n_pts, 3).")

    h_scale = cubic_features.size(2) / 2
    ptcloud = ptcloud * h_scale + h_scale
    return CubicFeatureSamplingFunction.apply(ptcloud, cubic_features, neighborhood_size)
