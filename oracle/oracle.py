"""ctypes/numpy front end of the CPU oracle (oracle_tpk.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke`` and by the
CPU-baseline legs of ``bench.py``; the shipped package never imports it.

Each function takes and returns numpy arrays (torch CPU tensors are accepted and
converted) with the dtypes the reference returns on its CUDA path:
FPS int32, ball query int64 idx + float32 squared dist, three_nn float32 squared
dist + int32 idx, kNN int64 idx + float32 squared dist, chamfer int32 idx.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_tpk.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)


def build():
    """Compile oracle_tpk.c with gcc (oracle/Makefile, target ``oracle``)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
            os.path.join(_HERE, "oracle_tpk.c")
        ):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_knn.restype = ctypes.c_int
        _lib.orc_opt_n_threads.restype = ctypes.c_int
    return _lib


def _np(a, dtype):
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=dtype)


def _p(a, t):
    return a.ctypes.data_as(t)


def opt_n_threads(n):
    return lib().orc_opt_n_threads(ctypes.c_int(int(n)))


def fps(xyz, npoint):
    xyz = _np(xyz, np.float32)
    b, n, _ = xyz.shape
    out = np.zeros((b, npoint), np.int32)
    lib().orc_fps(b, n, int(npoint), _p(xyz, _f32p), _p(out, _i32p))
    return out


def ball_query_dense(radius, nsample, x, y, return_pairs=False):
    """x (B,N,3) candidates, y (B,M,3) centres -> idx (B,M,ns) int64, dist2 (B,M,ns) f32."""
    x = _np(x, np.float32)
    y = _np(y, np.float32)
    b, n, _ = x.shape
    m = y.shape[1]
    idx = np.zeros((b, m, nsample), np.int64)
    dist = np.zeros((b, m, nsample), np.float32)
    pairs = ctypes.c_int64(0)
    lib().orc_ball_query_dense(b, n, m, ctypes.c_float(radius), int(nsample), _p(y, _f32p),
                               _p(x, _f32p), _p(idx, _i64p), _p(dist, _f32p), ctypes.byref(pairs))
    return (idx, dist, pairs.value) if return_pairs else (idx, dist)


def ball_query_partial(radius, nsample, x, y, batch_x, batch_y, return_pairs=False):
    x = _np(x, np.float32)
    y = _np(y, np.float32)
    bx = _np(batch_x, np.int64)
    by = _np(batch_y, np.int64)
    idx = np.zeros((y.shape[0], nsample), np.int64)
    dist = np.zeros((y.shape[0], nsample), np.float32)
    pairs = ctypes.c_int64(0)
    lib().orc_ball_query_partial(ctypes.c_int64(x.shape[0]), ctypes.c_int64(y.shape[0]),
                                 ctypes.c_float(radius), int(nsample), _p(x, _f32p), _p(y, _f32p),
                                 _p(bx, _i64p), _p(by, _i64p), _p(idx, _i64p), _p(dist, _f32p),
                                 ctypes.byref(pairs))
    return (idx, dist, pairs.value) if return_pairs else (idx, dist)


def three_nn(unknown, known):
    """Returns (dist2, idx): SQUARED distances, as the native reference call does."""
    unknown = _np(unknown, np.float32)
    known = _np(known, np.float32)
    b, n, _ = unknown.shape
    m = known.shape[1]
    d2 = np.zeros((b, n, 3), np.float32)
    idx = np.zeros((b, n, 3), np.int32)
    lib().orc_three_nn(b, n, m, _p(unknown, _f32p), _p(known, _f32p), _p(d2, _f32p), _p(idx, _i32p))
    return d2, idx


def knn(pos_support, pos, k):
    s = _np(pos_support, np.float32)
    q = _np(pos, np.float32)
    b, n, _ = s.shape
    m = q.shape[1]
    idx = np.zeros((b, m, k), np.int64)
    d2 = np.zeros((b, m, k), np.float32)
    rc = lib().orc_knn(b, n, m, int(k), _p(s, _f32p), _p(q, _f32p), _p(idx, _i64p), _p(d2, _f32p))
    if rc != 0:
        raise RuntimeError("Not enough points in support to find %d neighboors" % k)
    return idx, d2


def knn_segmented(pos_support, pos, batch_support, batch_pos, k):
    """Per-segment kNN on packed arrays: the reference's dense kNN applied to each
    segment on its own, indices shifted back into the packed support array."""
    s = _np(pos_support, np.float32)
    q = _np(pos, np.float32)
    bs = _np(batch_support, np.int64)
    bq = _np(batch_pos, np.int64)
    idx = np.full((q.shape[0], k), -1, np.int64)
    d2 = np.full((q.shape[0], k), -1, np.float32)
    for seg in np.unique(bq):
        s_lo, s_hi = np.searchsorted(bs, seg, "left"), np.searchsorted(bs, seg, "right")
        q_lo, q_hi = np.searchsorted(bq, seg, "left"), np.searchsorted(bq, seg, "right")
        kk = min(k, s_hi - s_lo)
        if kk == 0:
            continue
        i, d = knn(s[None, s_lo:s_hi], q[None, q_lo:q_hi], kk)
        idx[q_lo:q_hi, :kk] = i[0] + s_lo
        d2[q_lo:q_hi, :kk] = d[0]
    return idx, d2


def three_interpolate(features, idx, weight):
    f = _np(features, np.float32)
    idx = _np(idx, np.int32)
    w = _np(weight, np.float32)
    b, c, m = f.shape
    n = idx.shape[1]
    out = np.zeros((b, c, n), np.float32)
    lib().orc_three_interpolate(b, c, m, n, _p(f, _f32p), _p(idx, _i32p), _p(w, _f32p), _p(out, _f32p))
    return out


def three_interpolate_grad(grad_out, idx, weight, m):
    g = _np(grad_out, np.float32)
    idx = _np(idx, np.int32)
    w = _np(weight, np.float32)
    b, c, n = g.shape
    out = np.zeros((b, c, m), np.float32)
    lib().orc_three_interpolate_grad(b, c, n, int(m), _p(g, _f32p), _p(idx, _i32p), _p(w, _f32p),
                                     _p(out, _f32p))
    return out


def grouping(features, idx):
    f = _np(features, np.float32)
    idx = _np(idx, np.int64)
    b, c, n = f.shape
    _, npoint, nsample = idx.shape
    out = np.zeros((b, c, npoint, nsample), np.float32)
    lib().orc_grouping(b, c, n, npoint, nsample, _p(f, _f32p), _p(idx, _i64p), _p(out, _f32p))
    return out


def grouping_grad(grad_out, idx, n):
    g = _np(grad_out, np.float32)
    idx = _np(idx, np.int64)
    b, c, npoint, nsample = g.shape
    out = np.zeros((b, c, n), np.float32)
    lib().orc_grouping_grad(b, c, int(n), npoint, nsample, _p(g, _f32p), _p(idx, _i64p), _p(out, _f32p))
    return out


def chamfer(xyz1, xyz2):
    """Returns dist1 (B,n), dist2 (B,m), idx1, idx2 (int32), like the native reference call."""
    a = xyz1.detach().cpu().numpy() if hasattr(xyz1, "detach") else np.asarray(xyz1)
    if a.dtype == np.float64:
        x1 = _np(xyz1, np.float64)
        x2 = _np(xyz2, np.float64)
        fn, pt, dt = lib().orc_chamfer_dir_f64, _f64p, np.float64
    else:
        x1 = _np(xyz1, np.float32)
        x2 = _np(xyz2, np.float32)
        fn, pt, dt = lib().orc_chamfer_dir, _f32p, np.float32
    b, n, _ = x1.shape
    m = x2.shape[1]
    d1 = np.zeros((b, n), dt)
    d2 = np.zeros((b, m), dt)
    i1 = np.zeros((b, n), np.int32)
    i2 = np.zeros((b, m), np.int32)
    fn(b, n, _p(x1, pt), m, _p(x2, pt), _p(d1, pt), _p(i1, _i32p))
    fn(b, m, _p(x2, pt), n, _p(x1, pt), _p(d2, pt), _p(i2, _i32p))
    return d1, d2, i1, i2


def chamfer_grad(xyz1, xyz2, idx1, idx2, grad_dist1, grad_dist2):
    x1 = _np(xyz1, np.float32)
    x2 = _np(xyz2, np.float32)
    i1 = _np(idx1, np.int32)
    i2 = _np(idx2, np.int32)
    g1 = _np(grad_dist1, np.float32)
    g2 = _np(grad_dist2, np.float32)
    b, n, _ = x1.shape
    m = x2.shape[1]
    o1 = np.zeros_like(x1)
    o2 = np.zeros_like(x2)
    lib().orc_chamfer_grad(b, n, _p(x1, _f32p), m, _p(x2, _f32p), _p(i1, _i32p), _p(i2, _i32p),
                           _p(g1, _f32p), _p(g2, _f32p), _p(o1, _f32p), _p(o2, _f32p))
    return o1, o2


def grow_proximity(neighbours, min_cluster_size):
    """neighbours (N, nsample) int64 -> list of clusters (lists of indices in traversal order),
    as _grow_proximity_core of the reference returns them."""
    nb = _np(neighbours, np.int64)
    n, ns = nb.shape
    members = np.zeros(max(n, 1), np.int64)
    offsets = np.zeros(n + 2, np.int64)
    fn = lib().orc_grow_proximity
    fn.restype = ctypes.c_int64
    k = fn(ctypes.c_int64(n), int(ns), _p(nb, _i64p), ctypes.c_int64(int(min_cluster_size)), _p(members, _i64p),
           _p(offsets, _i64p))
    return [members[offsets[c]:offsets[c + 1]].tolist() for c in range(int(k))]


def instance_iou(num_gt, proposals_idx, proposals_offset, instance_labels, offset_num_gt, batch, instance_pointnum):
    """The native reference call (cuda/src/metrics.cpp:13-51) on numpy int64 arrays."""
    arrs = [_np(a, np.int64) for a in (num_gt, proposals_idx, proposals_offset, instance_labels, offset_num_gt, batch,
                                       instance_pointnum)]
    nprop = arrs[2].shape[0] - 1
    total = int(arrs[0].sum())
    out = np.zeros((nprop, total), np.float32)
    lib().orc_instance_iou(int(nprop), ctypes.c_int64(total), _p(arrs[0], _i64p), _p(arrs[1], _i64p), _p(arrs[2], _i64p),
                           _p(arrs[3], _i64p), _p(arrs[4], _i64p), _p(arrs[5], _i64p), _p(arrs[6], _i64p), _p(out, _f32p))
    return out


def gridding(ptcloud, scale):
    """ptcloud (B, n, 3) f32 in grid units -> grid (B, (2 scale)^3), weights (B, n, 8, 3), indexes (B, n, 8)."""
    p = _np(ptcloud, np.float32)
    b, n, _ = p.shape
    nv = (2 * scale) ** 3
    grid = np.zeros((b, nv), np.float32)
    w = np.zeros((b, n, 8, 3), np.float32)
    ix = np.zeros((b, n, 8), np.int32)
    f = ctypes.c_float
    lib().orc_gridding(b, n, f(-scale), f(scale - 1), f(-scale), f(scale - 1), f(-scale), f(scale - 1), _p(p, _f32p),
                       _p(grid, _f32p), _p(w, _f32p), _p(ix, _i32p))
    return grid, w, ix


def gridding_grad(weights, indexes, grad_grid):
    w = _np(weights, np.float32)
    ix = _np(indexes, np.int32)
    g = _np(grad_grid, np.float32)
    b, n = ix.shape[0], ix.shape[1]
    out = np.zeros((b, n, 3), np.float32)
    lib().orc_gridding_grad(b, n, ctypes.c_int64(g.shape[1]), _p(w, _f32p), _p(ix, _i32p), _p(g, _f32p), _p(out, _f32p))
    return out


def cubic_feature_sampling(ptcloud, cubic_features, neighborhood_size=1):
    """ptcloud (B, n, 3) f32 in grid units, cubic_features (B, c, s, s, s) -> features (B, n, nv, c), indexes (B, n, nv)."""
    p = _np(ptcloud, np.float32)
    cf = _np(cubic_features, np.float32)
    b, n, _ = p.shape
    c, s = cf.shape[1], cf.shape[2]
    nv = (2 * neighborhood_size) ** 3
    out = np.zeros((b, n, nv, c), np.float32)
    ix = np.zeros((b, n, nv), np.int32)
    lib().orc_cubic_feature_sampling(b, n, c, s, int(neighborhood_size), _p(p, _f32p), _p(cf, _f32p), _p(out, _f32p),
                                     _p(ix, _i32p))
    return out, ix


def cubic_feature_sampling_grad(grad_point_features, indexes, scale, neighborhood_size=1):
    g = _np(grad_point_features, np.float32)
    ix = _np(indexes, np.int32)
    b, n, nv, c = g.shape
    out = np.zeros((b, c, scale, scale, scale), np.float32)
    lib().orc_cubic_feature_sampling_grad(b, n, c, int(scale), int(neighborhood_size), _p(g, _f32p), _p(ix, _i32p),
                                          _p(out, _f32p))
    return out
