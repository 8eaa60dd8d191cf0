"""Gridding: point clouds to 3D density grids by trilinear weights (reference:
torch_points_kernels/gridding.py, kernels cuda/src/gridding_gpu.cu)."""
import torch

from . import _lib


def _suffix(t, what):
    _lib.check_cuda(t, what)
    if t.dtype == torch.float32:
        return "f32"
    if t.dtype == torch.float64:
        return "f64"
    raise RuntimeError("%s must be a float32 or float64 tensor" % what)


class GriddingFunction(torch.autograd.Function):
    """grid = gridding(ptcloud) on the cube [-scale, scale - 1]^3; ptcloud is in grid units."""

    @staticmethod
    def forward(ctx, ptcloud, scale):
        sfx = _suffix(ptcloud, "ptcloud")
        ptcloud = ptcloud.contiguous()
        b, n = ptcloud.shape[0], ptcloud.shape[1]
        length = 2 * int(scale)
        grid = torch.empty((b, length ** 3), dtype=ptcloud.dtype, device=ptcloud.device)
        weights = torch.empty((b, n, 8, 3), dtype=ptcloud.dtype, device=ptcloud.device)
        indexes = torch.empty((b, n, 8), dtype=torch.int32, device=ptcloud.device)
        with torch.cuda.device(ptcloud.device):
            _lib.call("tpk_gridding_" + sfx, b, n, float(-scale), float(scale - 1), float(-scale), float(scale - 1),
                      float(-scale), float(scale - 1), _lib.ptr(ptcloud), _lib.ptr(grid), _lib.ptr(weights),
                      _lib.ptr(indexes), _lib.stream_of(ptcloud))
        ctx.save_for_backward(weights, indexes)
        return grid

    @staticmethod
    def backward(ctx, grad_grid):
        weights, indexes = ctx.saved_tensors
        sfx = _suffix(weights, "grid_pt_weights")
        grad_grid = grad_grid.contiguous()
        b, n = indexes.shape[0], indexes.shape[1]
        grad_ptcloud = torch.empty((b, n, 3), dtype=weights.dtype, device=weights.device)
        with torch.cuda.device(weights.device):
            _lib.call("tpk_gridding_grad_" + sfx, b, n, grad_grid.shape[1], _lib.ptr(weights), _lib.ptr(indexes),
                      _lib.ptr(grad_grid), _lib.ptr(grad_ptcloud), _lib.stream_of(weights))
        return grad_ptcloud, None


def gridding(ptcloud, scale):
    r"""
    Converts the input point clouds into 3D grids by trilinear interpolcation.
    Please refer to https://arxiv.org/pdf/2006.03761 for more information

    Parameters
    ----------
    ptcloud : torch.Tensor (dtype=torch.float32)
        (B, n_pts, 3) B point clouds containing n_pts points
    scale : Int
        the resolution of the 3D grid

    Returns
    -------
    grid: torch.Tensor
        (B, scale, scale, scale): the grid of the resolution of scale * scale * scale
    """
    if len(ptcloud.shape) != 3 or ptcloud.size(2) != 3:
        raise ValueError("The input point cloud should be of size (B, n_pts, 3)")

    ptcloud = ptcloud * scale
    grids = []
    # points whose coordinates sum to zero are padding and are dropped, cloud by cloud
    # (reference: gridding.py:54-60)
    for p in torch.split(ptcloud, 1, dim=0):
        non_zeros = torch.sum(p, dim=2).ne(0)
        p = p[non_zeros].unsqueeze(dim=0)
        grids.append(GriddingFunction.apply(p, scale))
    return torch.cat(grids, dim=0).contiguous()
