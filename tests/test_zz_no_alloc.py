"""The allocation-free FPS entry point (tpk_furthest_point_sampling_static), called through
the C ABI exactly as a caller that may not allocate would: inputs and outputs are
buffers it already owns, nothing else is passed.  Its indices must equal those of the
regular entry point (which gets its scratch from the caller) on two calls in a row that
reuse the built-in scratch with different shapes.  Runs last so that a failure here
cannot hide any other test."""
import os

import numpy as np
import pytest
import torch

from torch_points_kernels_b200 import _lib
from tests import data

pytestmark = pytest.mark.gpu


def _regular(x, m):
    """The regular entry point steered onto the same kernel (large-cloud kernel, no sorted copy)
    through the library's test hook; the scratch is sized by the library for exactly that choice."""
    b, n = x.shape[0], x.shape[1]
    out = torch.empty((b, m), dtype=torch.int32, device=x.device)
    old = os.environ.get("TPK_B200_TEST")
    os.environ["TPK_B200_TEST"] = "fps_global,fps_unsorted"
    try:
        need = _lib.lib().tpk_fps_scratch_bytes(b, n, m)
        assert need == 4 * b * n
        scratch = torch.empty((need,), dtype=torch.uint8, device=x.device)
        _lib.call("tpk_furthest_point_sampling", b, n, m, _lib.ptr(x), _lib.ptr(scratch), need, _lib.ptr(out),
                  _lib.stream_of(x))
    finally:
        if old is None:
            os.environ.pop("TPK_B200_TEST", None)
        else:
            os.environ["TPK_B200_TEST"] = old
    return out


def _static(x, out, m):
    _lib.call("tpk_furthest_point_sampling_static", x.shape[0], x.shape[1], m, _lib.ptr(x), _lib.ptr(out),
              _lib.stream_of(x))


def test_static_scratch_entry_point_matches_regular_one_twice():
    dev = torch.device("cuda:0")
    cap = _lib.lib().tpk_fps_static_capacity()
    assert cap >= 1 << 20
    # every buffer the two calls need exists before the first of them
    x1 = data.gaussian_mixture(2, 150000, seed=71).to(dev)
    x2 = data.unit_ball(5, 3000, seed=72).to(dev)
    out1 = torch.empty((2, 40), dtype=torch.int32, device=dev)
    out2 = torch.empty((5, 257), dtype=torch.int32, device=dev)
    want1, want2 = _regular(x1, 40), _regular(x2, 257)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    _static(x1, out1, 40)
    _static(x2, out2, 257)     # reuses the scratch the first call left dirty
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    np.testing.assert_array_equal(out1.cpu().numpy(), want1.cpu().numpy())
    np.testing.assert_array_equal(out2.cpu().numpy(), want2.cpu().numpy())
    assert _lib.device_status() == 0


def test_static_scratch_entry_point_rejects_oversize():
    dev = torch.device("cuda:0")
    cap = _lib.lib().tpk_fps_static_capacity()
    x = torch.zeros((1, 8, 3), device=dev)
    out = torch.zeros((1, 4), dtype=torch.int32, device=dev)
    # sizes are checked before anything is launched: claim more points than the scratch holds
    rc = _lib.lib().tpk_furthest_point_sampling_static(2, int(cap // 2 + 1), 4, _lib.ptr(x), _lib.ptr(out),
                                                       _lib.stream_of(x))
    assert rc == 3
    assert b"exceed the built-in scratch" in _lib.lib().tpk_last_error()
