"""CPU tests of the drop-in boundary: the shared library loads and exports exactly what
include/tpk_b200.h declares, and the Python surface raises the reference's exceptions
without touching a GPU."""
import ctypes
import os
import re

import pytest
import torch

import torch_points_kernels_b200 as tpk
from torch_points_kernels_b200 import _lib, chamfer_dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "tpk_b200.h")).read()
    return sorted(set(re.findall(r"TPK_API\s+[\w\s\*]+?\b(tpk_\w+)\s*\(", text)))


def test_header_symbols_exported():
    names = _declared()
    assert len(names) >= 18
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), n
    assert sorted(_lib.EXPORTS) == names


def test_version_and_error_text():
    l = _lib.lib()
    assert l.tpk_version() >= 100
    assert isinstance(l.tpk_last_error(), bytes)


def test_invalid_arguments_return_status_without_gpu():
    l = _lib.lib()
    # argument validation happens before any CUDA call
    assert l.tpk_knn_dense(1, 3, 1, 5, None, None, None, None, None) == 1
    assert b"Not enough points" in l.tpk_last_error()
    assert l.tpk_ball_query_dense(-1, 1, 1, 0.1, 1, None, None, None, None, None) == 1
    assert l.tpk_three_nn(1, 4, 4, None, None, None, None, None) == 1
    assert l.tpk_furthest_point_sampling(1, 0, 2, None, None, 0, None, None) == 1
    # empty problems are no-ops
    assert l.tpk_furthest_point_sampling(0, 10, 2, None, None, 0, None, None) == 0
    assert l.tpk_grouping(0, 4, 4, 4, 4, None, None, None, None) == 0


def test_fps_refuses_short_scratch_without_gpu():
    """A scratch buffer smaller than tpk_fps_scratch_bytes is refused before anything is launched
    (the sizes are checked on the host; the pointers are never dereferenced)."""
    l = _lib.lib()
    need = l.tpk_fps_scratch_bytes(2, 200000, 48)
    assert need == 2 * 200000 * 20
    fake = ctypes.c_void_p(256)  # never dereferenced: the call fails on the size
    for fn, extra in ((l.tpk_furthest_point_sampling, ()), (l.tpk_furthest_point_sampling_xyz, (None,))):
        rc = fn(2, 200000, 48, fake, fake, need - 1, fake, *extra, None)
        assert rc == 4  # TPK_ERR_SCRATCH
        assert b"scratch of" in l.tpk_last_error()
    # optional scratch (sorted copy of a cloud that fits on chip) is checked the same way
    need = l.tpk_fps_scratch_bytes(16, 16384, 4096)
    assert l.tpk_furthest_point_sampling(16, 16384, 4096, fake, fake, need // 2, fake, None) == 4
    # and a missing buffer where one is required
    assert l.tpk_furthest_point_sampling(2, 200000, 48, fake, None, 0, fake, None) == 4


def test_scratch_sizes_are_host_arithmetic(monkeypatch):
    """What the callers must allocate: pure host functions, usable without a GPU."""
    monkeypatch.delenv("TPK_B200_TEST", raising=False)
    l = _lib.lib()
    # FPS: nothing for small clouds or few samples, the sorted copy (16 B/point) for clouds that stay
    # on chip, the sorted copy plus the running minima (20 B/point) above 131072 points
    assert l.tpk_fps_scratch_bytes(4, 1024, 256) == 0
    assert l.tpk_fps_scratch_bytes(4, 16384, 64) == 0
    assert l.tpk_fps_scratch_bytes(16, 16384, 4096) == 16 * 16384 * 16
    assert l.tpk_fps_scratch_bytes(2, 200000, 48) == 2 * 200000 * 20
    monkeypatch.setenv("TPK_B200_TEST", "fps_unsorted")
    assert l.tpk_fps_scratch_bytes(16, 16384, 4096) == 0
    assert l.tpk_fps_scratch_bytes(2, 200000, 48) == 2 * 200000 * 4
    monkeypatch.setenv("TPK_B200_TEST", "ball_query_scan,fps_global,fps_config=2:64:8")
    assert l.tpk_fps_scratch_bytes(2, 1000, 48) == 2 * 1000 * 20
    assert l.tpk_ball_query_dense_scratch_bytes(16, 16384, 4096, 32) == 0
    monkeypatch.delenv("TPK_B200_TEST")
    # ball query: one flag per centre with the grid in shared memory, the whole grid for huge clouds
    assert l.tpk_ball_query_dense_scratch_bytes(2, 256, 64, 32) == 0
    assert l.tpk_ball_query_dense_scratch_bytes(16, 16384, 4096, 32) == 16 * 4096
    assert l.tpk_ball_query_dense_scratch_bytes(2, 300000, 100, 32) > 2 * 300000 * 16
    # packed ball query: buckets, sorted copy (20 B/point) and one flag per query from 4096 points on
    assert l.tpk_ball_query_partial_dense_scratch_bytes(1000, 100, 0.1) == 0
    assert l.tpk_ball_query_partial_dense_scratch_bytes(100000, 5000, 0.1) > 100000 * 20 + 5000
    assert l.tpk_ball_query_partial_dense_scratch_bytes(100000, 5000, 0.0) == 0
    # three_nn: one flag per unknown point (grid in shared memory), the whole grid for huge known clouds
    assert l.tpk_three_nn_scratch_bytes(2, 256, 64) == 0
    assert l.tpk_three_nn_scratch_bytes(16, 16384, 4096) == 16 * 16384
    assert l.tpk_three_nn_scratch_bytes(2, 3000, 10000) == (2 * 3000 + 255) // 256 * 256
    assert l.tpk_three_nn_scratch_bytes(1, 1000, 3000000) > 3000000 * 16
    # chamfer: flags for the larger direction
    assert l.tpk_chamfer_dist_scratch_bytes(4, 512, 700) == 0
    assert l.tpk_chamfer_dist_scratch_bytes(32, 16384, 16384) == 32 * 16384
    assert l.tpk_three_nn_scratch_bytes(0, 10, 10) == 0
    assert _lib.kernel_launches() >= 0


def test_python_surface_matches_reference_names():
    for name in ("ball_query", "furthest_point_sample", "grouping_operation", "three_interpolate",
                 "three_nn", "knn"):
        assert callable(getattr(tpk, name))
    assert callable(chamfer_dist.chamfer_dist) and hasattr(chamfer_dist, "ChamferFunction")


def test_python_level_errors():
    x = torch.rand(2, 16, 3)
    with pytest.raises(ValueError):
        tpk.furthest_point_sample(x, 17)
    with pytest.raises(ValueError):
        tpk.three_nn(torch.rand(2, 2, 3), x)
    with pytest.raises(Exception):
        tpk.ball_query(0.1, 4, x, x, mode=None)
    with pytest.raises(Exception):
        tpk.ball_query(0.1, 4, x, x, mode="sparse")
    with pytest.raises(Exception):
        tpk.ball_query(0.1, 4, x, x, mode="dense", batch_x=torch.zeros(2))
    with pytest.raises(Exception):
        tpk.ball_query(0.1, 4, x[0], x[0], mode="PARTIAL_DENSE")
    with pytest.raises(NotImplementedError):
        tpk.ball_query(0.1, 4, x, x, sort=True)
    with pytest.raises(ValueError):
        chamfer_dist.chamfer_dist(torch.rand(2, 3), torch.rand(2, 5, 3))
    with pytest.raises(AssertionError):
        tpk.ball_query(0.1, 4, x, x, mode="partial_dense", batch_x=torch.zeros(2, dtype=torch.long),
                       batch_y=torch.zeros(2, dtype=torch.long))


def test_cpu_tensors_are_rejected_not_silently_computed():
    # no CPU fallback: the reference's CHECK_CUDA message, as a RuntimeError
    x = torch.rand(2, 16, 3)
    for fn in (lambda: tpk.furthest_point_sample(x, 4), lambda: tpk.three_nn(x, x),
               lambda: tpk.ball_query(0.1, 4, x, x), lambda: tpk.knn(x, x, 2),
               lambda: tpk.grouping_operation(torch.rand(2, 3, 16), torch.zeros(2, 4, 2, dtype=torch.long)),
               lambda: chamfer_dist.chamfer_dist(x, x)):
        with pytest.raises(RuntimeError, match="CUDA tensor"):
            fn()


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libtpk_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_segment_vectors_are_validated_like_the_reference_cpu_path(known_answers):
    """The reference's CPU path raises RuntimeError when batch_x and batch_y name different
    numbers of segments (its own test vector); the same check, plus sortedness, is what the
    wrappers run under TPK_B200_DEBUG.  The check itself needs no GPU."""
    ka = known_answers["ball_query_partial_segment_mismatch"]
    bx, by = torch.tensor(ka["batch_x"]), torch.tensor(ka["batch_y"])
    with pytest.raises(RuntimeError, match="same number of samples"):
        _lib.check_segments(bx, by)
    _lib.check_segments(torch.tensor([0, 0, 1, 1]), torch.tensor([0, 1]))
    with pytest.raises(RuntimeError, match="sorted"):
        _lib.check_segments(torch.tensor([0, 1, 0, 1]), torch.tensor([0, 1]))
    with pytest.raises(RuntimeError, match="sorted"):
        _lib.check_segments(torch.tensor([0, 1]), torch.tensor([-1, 1]))
    _lib.check_segments(torch.tensor([], dtype=torch.long), torch.tensor([], dtype=torch.long))


def test_grouping_grad_scratch_is_sized_and_checked():
    """The sorted backward (rows of more than 32 KB) asks for 4 bytes per position, padded to whole
    tiles, and refuses a shorter buffer before anything is launched; other shapes ask for nothing."""
    l = _lib.lib()
    assert l.tpk_grouping_grad_scratch_bytes(16, 64, 16384, 4096, 32) == 16 * 4096 * 32 * 4
    assert l.tpk_grouping_grad_scratch_bytes(2, 8, 10000, 100, 3) == 2 * 512 * 4   # 300 positions, one tile of 512
    assert l.tpk_grouping_grad_scratch_bytes(2, 8, 4096, 1024, 32) == 0           # short rows: the atomic kernels
    assert l.tpk_grouping_grad_scratch_bytes(1, 3, 60000, 500, 16) == 0           # the row does not fit shared memory
    assert l.tpk_grouping_grad_scratch_bytes(0, 3, 10000, 5, 1) == 0
    rc = l.tpk_grouping_grad_ws(2, 8, 10000, 100, 3, ctypes.c_void_p(256), ctypes.c_void_p(256), ctypes.c_void_p(256),
                                ctypes.c_void_p(256), ctypes.c_int64(100), None)
    assert rc == 4 and b"scratch" in l.tpk_last_error()


def test_test_hook_tokens(monkeypatch):
    """TPK_B200_TEST is a comma-separated token list; a token only matches whole names."""
    l = _lib.lib()
    monkeypatch.setenv("TPK_B200_TEST", "fps_unsortedx,xfps_unsorted")
    assert l.tpk_fps_scratch_bytes(16, 16384, 4096) == 16 * 16384 * 16
    monkeypatch.setenv("TPK_B200_TEST", "three_nn_scan,fps_unsorted")
    assert l.tpk_fps_scratch_bytes(16, 16384, 4096) == 0
    assert l.tpk_three_nn_scratch_bytes(16, 16384, 4096) == 0
    monkeypatch.delenv("TPK_B200_TEST")
    assert l.tpk_three_nn_scratch_bytes(16, 16384, 4096) > 0
