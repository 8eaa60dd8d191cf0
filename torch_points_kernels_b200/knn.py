"""k nearest neighbours on the GPU.

The reference implements kNN on the CPU only and raises on CUDA tensors
(torch_points_kernels/knn.py:4-18); here the same call runs a brute-force sm_100a
kernel with the CPU path's arithmetic (unfused squared distance) and result order.
"""
import torch

from . import _lib


def knn(pos_support, pos, k, batch_support=None, batch_pos=None):
    """kNN search.

    Dense layout (the reference's only one):
        pos_support - [B,N,3] support points
        pos - [B,M,3] centre of queries
        k - number of neighboors, needs to be <= N
        returns idx [B,M,k] int64, dist2 [B,M,k] float32 squared distances, ascending

    Packed layout (extension, when batch_support and batch_pos are given):
        pos_support - [N,3], pos - [M,3], batch_* - sorted int64 segment ids
        returns idx [M,k] (positions in pos_support) and dist2 [M,k]; a query whose
        segment holds fewer than k support points has -1 in the missing slots
    """
    for t, name in ((pos_support, "support"), (pos, "query")):
        _lib.check_contiguous(t, name)
        _lib.check_cuda(t, name)
        if t.dtype != torch.float32:
            raise RuntimeError("%s must be a float32 tensor" % name)
    if (batch_support is None) != (batch_pos is None):
        raise Exception("batch_support and batch_pos should be provided together")
    if batch_support is None:
        assert pos_support.dim() == 3 and pos.dim() == 3
        b, n = pos_support.shape[0], pos_support.shape[1]
        m = pos.shape[1]
        if n < k:
            raise RuntimeError("Not enough points in support to find " + str(k) + " neighboors")
        idx = torch.empty((b, m, k), dtype=torch.int64, device=pos.device)
        dist2 = torch.empty((b, m, k), dtype=torch.float32, device=pos.device)
        with torch.cuda.device(pos.device):
            need = _lib.lib().tpk_knn_dense_scratch_bytes(b, n, m, int(k))
            if need > 0:
                # large clouds: hashed uniform grid with scratch (same results as the scan)
                scratch = torch.empty((need,), dtype=torch.uint8, device=pos.device)
                _lib.call("tpk_knn_dense_ws", b, n, m, int(k), _lib.ptr(pos_support), _lib.ptr(pos),
                          _lib.ptr(idx), _lib.ptr(dist2), _lib.ptr(scratch), need, _lib.stream_of(pos))
            else:
                _lib.call("tpk_knn_dense", b, n, m, int(k), _lib.ptr(pos_support), _lib.ptr(pos),
                          _lib.ptr(idx), _lib.ptr(dist2), _lib.stream_of(pos))
        return idx, dist2

    assert pos_support.dim() == 2 and pos.dim() == 2
    assert pos_support.size(0) == batch_support.size(0)
    assert pos.size(0) == batch_pos.size(0)
    for t, name in ((batch_support, "batch_support"), (batch_pos, "batch_pos")):
        _lib.check_cuda(t, name)
        if t.dtype != torch.int64:
            raise RuntimeError("%s must be an int64 tensor" % name)
    batch_support = batch_support.contiguous()
    batch_pos = batch_pos.contiguous()
    if _lib.debug_checks():
        _lib.check_segments(batch_support, batch_pos)
    m = pos.shape[0]
    idx = torch.empty((m, k), dtype=torch.int64, device=pos.device)
    dist2 = torch.empty((m, k), dtype=torch.float32, device=pos.device)
    with torch.cuda.device(pos.device):
        need = _lib.lib().tpk_knn_partial_dense_scratch_bytes(pos_support.shape[0], m, int(k))
        if need > 0:
            scratch = torch.empty((need,), dtype=torch.uint8, device=pos.device)
            _lib.call("tpk_knn_partial_dense_ws", pos_support.shape[0], m, int(k), _lib.ptr(pos_support),
                      _lib.ptr(pos), _lib.ptr(batch_support), _lib.ptr(batch_pos), _lib.ptr(idx),
                      _lib.ptr(dist2), _lib.ptr(scratch), need, _lib.stream_of(pos))
        else:
            _lib.call("tpk_knn_partial_dense", pos_support.shape[0], m, int(k), _lib.ptr(pos_support),
                      _lib.ptr(pos), _lib.ptr(batch_support), _lib.ptr(batch_pos), _lib.ptr(idx),
                      _lib.ptr(dist2), _lib.stream_of(pos))
    return idx, dist2
