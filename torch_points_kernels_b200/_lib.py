"""Loader of the C-ABI CUDA library (libtpk_b200.so) and thin tensor-to-pointer glue.

The library is the only implementation of every op in this package: there is no CPU
or pure-PyTorch fallback.  If it is missing, importing an op fails with a clear error.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# TPK_B200_LIB points at another build of the library (e.g. one made with different tuning flags)
LIB_PATH = os.environ.get("TPK_B200_LIB") or os.path.join(_HERE, "libtpk_b200.so")

_lib = None

_c_int = ctypes.c_int
_c_i64 = ctypes.c_int64
_c_f32 = ctypes.c_float
_ptr = ctypes.c_void_p

# name -> argument types, in the order of include/tpk_b200.h
_SIGNATURES = {
    "tpk_furthest_point_sampling": [_c_int, _c_int, _c_int, _ptr, _ptr, _c_i64, _ptr, _ptr],
    "tpk_furthest_point_sampling_xyz": [_c_int, _c_int, _c_int, _ptr, _ptr, _c_i64, _ptr, _ptr, _ptr],
    "tpk_furthest_point_sampling_static": [_c_int, _c_int, _c_int, _ptr, _ptr, _ptr],
    "tpk_ball_query_dense": [_c_int, _c_int, _c_int, _c_f32, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_ball_query_dense_ws": [_c_int, _c_int, _c_int, _c_f32, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr],
    "tpk_ball_query_partial_dense": [_c_i64, _c_i64, _c_f32, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_ball_query_partial_dense_ws": [_c_i64, _c_i64, _c_f32, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                                        _c_i64, _ptr],
    "tpk_three_nn": [_c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_chamfer_dist_f32_ws": [_c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr],
    "tpk_three_nn_ws": [_c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr],
    "tpk_knn_dense": [_c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_knn_partial_dense": [_c_i64, _c_i64, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_knn_dense_ws": [_c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr],
    "tpk_knn_partial_dense_ws": [_c_i64, _c_i64, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr],
    "tpk_three_interpolate": [_c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_three_interpolate_grad": [_c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_grouping": [_c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr],
    "tpk_grouping_grad": [_c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr],
    "tpk_grouping_grad_ws": [_c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr],
    "tpk_sa_group_grad": [_c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr],
    "tpk_chamfer_dist_f32": [_c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_chamfer_dist_f64": [_c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_chamfer_dist_grad_f32": [_c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_chamfer_dist_grad_f64": [_c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_gridding_f32": [_c_int, _c_int, _c_f32, _c_f32, _c_f32, _c_f32, _c_f32, _c_f32, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_gridding_f64": [_c_int, _c_int, _c_f32, _c_f32, _c_f32, _c_f32, _c_f32, _c_f32, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_gridding_grad_f32": [_c_int, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_gridding_grad_f64": [_c_int, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_cubic_feature_sampling_f32": [_c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_cubic_feature_sampling_f64": [_c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_cubic_feature_sampling_grad_f32": [_c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_cubic_feature_sampling_grad_f64": [_c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr],
    "tpk_sa_group": [_c_int, _c_int, _c_int, _c_int, _c_f32, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr],
    "tpk_grow_labels_step": [_c_i64, _c_int, _ptr, _ptr, _ptr, _c_int, _ptr],
    "tpk_instance_iou": [_c_int, _c_i64, _c_i64, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
}

EXPORTS = sorted(list(_SIGNATURES) + ["tpk_version", "tpk_last_error", "tpk_device_status", "tpk_kernel_launches", "tpk_fps_scratch_bytes",
                                       "tpk_fps_static_capacity", "tpk_ball_query_dense_scratch_bytes",
                                       "tpk_three_nn_scratch_bytes", "tpk_chamfer_dist_scratch_bytes",
                                       "tpk_ball_query_partial_dense_scratch_bytes", "tpk_knn_dense_scratch_bytes", "tpk_sa_group_scratch_bytes",
                                       "tpk_knn_partial_dense_scratch_bytes", "tpk_grouping_grad_scratch_bytes"])


def lib():
    """Returns the loaded library, loading it on first use."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "torch_points_kernels_b200: %s is missing. Build it with "
                "`make -C torch_points_kernels_b200/csrc` (needs nvcc with sm_100a support); "
                "this package has no CPU or PyTorch fallback." % LIB_PATH
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = _c_int
        handle.tpk_version.restype = _c_int
        handle.tpk_last_error.restype = ctypes.c_char_p
        handle.tpk_kernel_launches.argtypes = []
        handle.tpk_kernel_launches.restype = _c_i64
        handle.tpk_device_status.argtypes = [ctypes.POINTER(_c_int), _c_int]
        handle.tpk_device_status.restype = _c_int
        handle.tpk_fps_scratch_bytes.argtypes = [_c_int, _c_int, _c_int]
        handle.tpk_fps_scratch_bytes.restype = _c_i64
        handle.tpk_ball_query_dense_scratch_bytes.argtypes = [_c_int, _c_int, _c_int, _c_int]
        handle.tpk_ball_query_dense_scratch_bytes.restype = _c_i64
        handle.tpk_ball_query_partial_dense_scratch_bytes.argtypes = [_c_i64, _c_i64, _c_f32]
        handle.tpk_ball_query_partial_dense_scratch_bytes.restype = _c_i64
        handle.tpk_chamfer_dist_scratch_bytes.argtypes = [_c_int, _c_int, _c_int]
        handle.tpk_chamfer_dist_scratch_bytes.restype = _c_i64
        handle.tpk_three_nn_scratch_bytes.argtypes = [_c_int, _c_int, _c_int]
        handle.tpk_three_nn_scratch_bytes.restype = _c_i64
        handle.tpk_knn_dense_scratch_bytes.argtypes = [_c_int, _c_int, _c_int, _c_int]
        handle.tpk_knn_dense_scratch_bytes.restype = _c_i64
        handle.tpk_knn_partial_dense_scratch_bytes.argtypes = [_c_i64, _c_i64, _c_int]
        handle.tpk_knn_partial_dense_scratch_bytes.restype = _c_i64
        handle.tpk_sa_group_scratch_bytes.argtypes = [_c_int, _c_int, _c_int, _c_int]
        handle.tpk_sa_group_scratch_bytes.restype = _c_i64
        handle.tpk_grouping_grad_scratch_bytes.argtypes = [_c_int, _c_int, _c_int, _c_int, _c_int]
        handle.tpk_grouping_grad_scratch_bytes.restype = _c_i64
        handle.tpk_fps_static_capacity.argtypes = []
        handle.tpk_fps_static_capacity.restype = _c_i64
        _lib = handle
    return _lib


def call(name, *args):
    """Calls an entry point; a non-zero status becomes a RuntimeError with the library's text."""
    handle = lib()
    status = getattr(handle, name)(*args)
    if status != 0:
        raise RuntimeError(handle.tpk_last_error().decode("utf-8", "replace") or "%s failed (%d)" % (name, status))


def stream_of(t):
    """The caller's current stream on the tensor's device, as the void* the C ABI takes."""
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() > 0 else ctypes.c_void_p(0)


def check_cuda(t, name):
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)


def check_contiguous(t, name):
    if not t.is_contiguous():
        raise RuntimeError("%s must be a contiguous tensor" % name)


def check_float(t, name):
    if not t.is_floating_point():
        raise RuntimeError("%s must be a float tensor" % name)


def check_int(t, name):
    if t.is_floating_point() or t.is_complex() or t.dtype == torch.bool:
        raise RuntimeError("%s must be an int tensor" % name)


def debug_checks():
    """True when TPK_B200_DEBUG is set to anything but 0: the wrappers then validate what the
    kernels take on trust (segment vectors) at the price of a device-to-host copy, and read
    the device status word after every call."""
    return os.environ.get("TPK_B200_DEBUG", "0") not in ("", "0")


def check_segments(batch_x, batch_y):
    """What the reference's CPU path verifies about packed batches (cpu/src/ball_query.cpp:86-88:
    both vectors name the same number of segments) plus what every implementation assumes
    (segment ids sorted ascending, non-negative).  Works on tensors of any device; on CUDA
    tensors it synchronises, which is why the wrappers only call it under TPK_B200_DEBUG."""
    for t, name in ((batch_x, "batch_x"), (batch_y, "batch_y")):
        if t.numel() == 0:
            continue
        if bool((t[1:] < t[:-1]).any()) or int(t[0]) < 0:
            raise RuntimeError("%s must hold sorted, non-negative segment ids" % name)
    if batch_x.numel() and batch_y.numel() and int(batch_x[-1]) != int(batch_y[-1]):
        raise RuntimeError("Both batches need to have the same number of samples.")


def raise_on_device_status(what):
    """Debug mode: turn a non-zero device status word into an exception right after the call."""
    v = device_status()
    if v & 2:
        raise RuntimeError("%s: an index outside its tensor was skipped" % what)
    if v & 1:
        raise RuntimeError("%s: a kernel gave up a bounded wait" % what)


def device_status(reset=True):
    """Sticky device-side status word (non-zero after a kernel gave up a bounded wait)."""
    out = _c_int(0)
    status = lib().tpk_device_status(ctypes.byref(out), 1 if reset else 0)
    if status != 0:
        raise RuntimeError(lib().tpk_last_error().decode("utf-8", "replace"))
    return out.value


def kernel_launches():
    """Kernels the library has launched (or recorded into a stream capture) in this process."""
    return int(lib().tpk_kernel_launches())
