"""Chamfer distance (reference: torch_points_kernels/chamfer_dist.py)."""
import torch

from . import _lib


class ChamferFunction(torch.autograd.Function):
    """Nearest-neighbour squared distances in both directions; float32 or float64."""

    @staticmethod
    def forward(ctx, xyz1, xyz2):
        for t, name in ((xyz1, "xyz1"), (xyz2, "xyz2")):
            _lib.check_cuda(t, name)
        if xyz1.dtype != xyz2.dtype or xyz1.dtype not in (torch.float32, torch.float64):
            raise RuntimeError("xyz1 and xyz2 must both be float32 or both float64")
        xyz1 = xyz1.contiguous()
        xyz2 = xyz2.contiguous()
        b, n = xyz1.shape[0], xyz1.shape[1]
        m = xyz2.shape[1]
        dist1 = torch.empty((b, n), dtype=xyz1.dtype, device=xyz1.device)
        dist2 = torch.empty((b, m), dtype=xyz1.dtype, device=xyz1.device)
        idx1 = torch.empty((b, n), dtype=torch.int32, device=xyz1.device)
        idx2 = torch.empty((b, m), dtype=torch.int32, device=xyz1.device)
        name = "tpk_chamfer_dist_f32" if xyz1.dtype == torch.float32 else "tpk_chamfer_dist_f64"
        with torch.cuda.device(xyz1.device):
            need = _lib.lib().tpk_chamfer_dist_scratch_bytes(b, n, m) if xyz1.dtype == torch.float32 else 0
            if need > 0:
                # large clouds: nearest neighbours on a uniform grid (same results as the all-pairs scan)
                scratch = torch.empty((need,), dtype=torch.uint8, device=xyz1.device)
                _lib.call("tpk_chamfer_dist_f32_ws", b, n, _lib.ptr(xyz1), m, _lib.ptr(xyz2), _lib.ptr(dist1),
                          _lib.ptr(dist2), _lib.ptr(idx1), _lib.ptr(idx2), _lib.ptr(scratch), need,
                          _lib.stream_of(xyz1))
            else:
                _lib.call(name, b, n, _lib.ptr(xyz1), m, _lib.ptr(xyz2), _lib.ptr(dist1), _lib.ptr(dist2),
                          _lib.ptr(idx1), _lib.ptr(idx2), _lib.stream_of(xyz1))
        ctx.save_for_backward(xyz1, xyz2, idx1, idx2)
        return dist1, dist2

    @staticmethod
    def backward(ctx, grad_dist1, grad_dist2):
        xyz1, xyz2, idx1, idx2 = ctx.saved_tensors
        grad_dist1 = grad_dist1.contiguous()
        grad_dist2 = grad_dist2.contiguous()
        b, n = xyz1.shape[0], xyz1.shape[1]
        m = xyz2.shape[1]
        grad_xyz1 = torch.empty_like(xyz1)
        grad_xyz2 = torch.empty_like(xyz2)
        name = "tpk_chamfer_dist_grad_f32" if xyz1.dtype == torch.float32 else "tpk_chamfer_dist_grad_f64"
        with torch.cuda.device(xyz1.device):
            _lib.call(name, b, n, _lib.ptr(xyz1), m, _lib.ptr(xyz2), _lib.ptr(idx1), _lib.ptr(idx2),
                      _lib.ptr(grad_dist1), _lib.ptr(grad_dist2), _lib.ptr(grad_xyz1),
                      _lib.ptr(grad_xyz2), _lib.stream_of(xyz1))
        return grad_xyz1, grad_xyz2


def chamfer_dist(xyz1, xyz2, ignore_zeros=False):
    r"""
    Calcuates the distance between B pairs of point clouds

    Parameters
    ----------
    xyz1 : torch.Tensor (dtype=torch.float32)
        (B, n1, 3) B point clouds containing n1 points
    xyz2 : torch.Tensor (dtype=torch.float32)
        (B, n2, 3) B point clouds containing n2 points
    ignore_zeros : bool
        ignore the point whose coordinate is (0, 0, 0) or not (only honoured for B == 1,
        as in the reference)

    Returns
    -------
    dist: torch.Tensor
        0-dim tensor: mean over all points of cloud 1 of the squared distance to the
        nearest point of cloud 2, plus the same with the clouds swapped
    """
    if len(xyz1.shape) != 3 or xyz1.size(2) != 3 or len(xyz2.shape) != 3 or xyz2.size(2) != 3:
        raise ValueError("The input point cloud should be of size (B, n_pts, 3)")

    batch_size = xyz1.size(0)
    if batch_size == 1 and ignore_zeros:
        non_zeros1 = torch.sum(xyz1, dim=2).ne(0)
        non_zeros2 = torch.sum(xyz2, dim=2).ne(0)
        xyz1 = xyz1[non_zeros1].unsqueeze(dim=0)
        xyz2 = xyz2[non_zeros2].unsqueeze(dim=0)

    dist1, dist2 = ChamferFunction.apply(xyz1, xyz2)
    return torch.mean(dist1) + torch.mean(dist2)
