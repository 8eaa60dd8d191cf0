"""GPU parity tests: every op, called through the Python surface (which calls the C ABI),
against the CPU oracle on the same seeded inputs.  Integer outputs and the distances the
search kernels return are compared bit for bit; interpolated / grouped values to 1e-5
relative; atomically accumulated gradients to 1e-4."""
import os

import numpy as np
import pytest
import torch

import torch_points_kernels_b200 as tpk
from torch_points_kernels_b200 import _lib, chamfer_dist as cd
from oracle import oracle as orc
from tests import data

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.int32)


def same_bits(got, want):
    np.testing.assert_array_equal(bits(got), bits(want))


def cu(t):
    return torch.as_tensor(t).to(DEV).contiguous()


def npy(t):
    return t.detach().cpu().numpy()


def _guarded(fn):
    """Runs fn, returns the device status word it left (and clears it)."""
    assert _lib.device_status() == 0
    out = fn()
    torch.cuda.synchronize()
    return out, _lib.device_status()


# ------------------------------------------------------------------------------ FPS

# kernel families of FPS on a cloud that stays on chip: without the spatially sorted copy, with it
# and one sample per exchange, with it and several samples per exchange (the default)
FPS_FAMILIES = ["fps_unsorted", "fps_sorted,fps_single", "fps_sorted"]


def test_fps_known_answer(known_answers):
    ka = known_answers["fps_start0"]
    out = tpk.furthest_point_sample(cu(np.asarray(ka["points"], np.float32)), ka["npoint"])
    assert out.dtype == torch.int32 and npy(out).tolist() == ka["idx"]


@pytest.mark.parametrize("B,N,m", [(3, 1000, 200), (2, 4096, 512), (2, 16384, 700), (1, 40000, 150),
                                   (1, 100000, 40), (4, 257, 257), (2, 31, 9), (5, 1, 1), (2, 2, 2)])
@pytest.mark.parametrize("family", FPS_FAMILIES)
def test_fps_matches_oracle(B, N, m, family, monkeypatch):
    data.use_paths(monkeypatch, family)
    x = data.unit_ball(B, N, seed=2000 + N)
    got = npy(tpk.furthest_point_sample(cu(x), m))
    np.testing.assert_array_equal(got, orc.fps(x, m))
    assert _lib.device_status() == 0


@pytest.mark.parametrize("cfg", ["1,128,32", "1,512,8", "1,256,16", "2,64,32", "2,512,4", "4,64,16",
                                 "4,256,4", "8,128,4", "8,64,8", "8,512,1", "16,64,4", "16,512,1",
                                 "16,128,2"])
def test_fps_every_cluster_shape(cfg, monkeypatch):
    """Same cloud through every cluster size / block size (cluster x threads x points per thread),
    with the flat and with the three-stage exchange."""
    x = data.unit_ball(3, 4000, seed=77)
    want = orc.fps(x, 300)
    for tree in (None, "fps_tree"):
        for family in FPS_FAMILIES:
            data.use_paths(monkeypatch, "fps_config=" + cfg.replace(",", ":"), tree, family)
            got = npy(tpk.furthest_point_sample(cu(x), 300))
            np.testing.assert_array_equal(got, want)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("n", [3, 8, 37, 64, 300, 700, 1000, 1500, 2048, 5000])
def test_fps_tie_break_and_skip_rule(n, monkeypatch):
    rng = np.random.default_rng(n)
    pts = np.zeros((2, n, 3), np.float32)
    pts[:, 0] = (1.0, 1.0, 1.0)
    pts[:, 1:] = (1.0, 1.0, 1.5)
    far = rng.choice(np.arange(1, n), size=max(1, (n - 1) // 2), replace=False)
    pts[0, far] = (5.0, 1.0, 1.0)          # many exact ties for the second sample
    pts[1, 1:] = rng.integers(0, 3, size=(n - 1, 3)).astype(np.float32)  # lattice: ties and skipped origin points
    m = min(n, 12)
    want = orc.fps(pts, m)
    # with fewer than bs threads per cluster a thread owns several residues of k mod bs
    for cfg in (None, "1:64:32", "2:64:32", "2:256:16", "4:128:16", "1:128:8", "2:64:4"):
        for family in FPS_FAMILIES:
            data.use_paths(monkeypatch, cfg and "fps_config=" + cfg, family)
            np.testing.assert_array_equal(npy(tpk.furthest_point_sample(cu(pts), m)), want)


def test_fps_sorted_copy_is_the_default_for_big_on_chip_clouds(monkeypatch):
    data.use_paths(monkeypatch)
    assert _lib.lib().tpk_fps_scratch_bytes(4, 16384, 4096) == 4 * 16384 * 16
    assert _lib.lib().tpk_fps_scratch_bytes(4, 1024, 256) == 0


@pytest.mark.parametrize("kind", ["clustered", "lattice", "planar", "nonfinite", "many_skipped"])
@pytest.mark.parametrize("family", ["fps_sorted", "fps_sorted,fps_single", "fps_sorted,fps_global"])
def test_fps_sorted_copy_hard_clouds(kind, family, monkeypatch):
    """Warp and chunk skipping must never change a result: crowded cells, exact ties everywhere,
    a collapsed axis, coordinates that are not finite, and points the skip rule excludes.
    All kernels that skip: the register-resident ones (several samples per exchange, one sample
    per exchange) and the one for large clouds."""
    data.use_paths(monkeypatch, family)
    rng = np.random.default_rng(len(kind))
    B, n, m = 2, 6000, 400
    if kind == "clustered":
        x = (rng.standard_normal((B, n, 3)) * 0.02 + rng.integers(0, 4, (B, n, 1)) * 2.0).astype(np.float32)
    elif kind == "lattice":
        x = rng.integers(0, 9, (B, n, 3)).astype(np.float32) / 4
    elif kind == "planar":
        x = rng.uniform(-1, 1, (B, n, 3)).astype(np.float32)
        x[..., 1] = 0.5
    elif kind == "nonfinite":
        x = data.unit_ball(B, n, seed=5).numpy().copy()
        x[0, 17, 0] = np.inf
        x[0, 400, 2] = np.nan
        x[1, 3000] = (-np.inf, 0.0, np.nan)
        m = 60
    else:
        x = data.unit_ball(B, n, seed=6).numpy().copy()
        x[:, 1::2] *= 0.01  # |p|^2 <= 1e-3: never candidates
    got = npy(tpk.furthest_point_sample(cu(x), m))
    np.testing.assert_array_equal(got, orc.fps(x, m))
    assert _lib.device_status() == 0


@pytest.mark.parametrize("B,N,m", [(2, 200000, 48), (3, 140000, 33), (1, 1200000, 20)])
@pytest.mark.parametrize("sorted_copy", ["1", "0"])
def test_fps_large_clouds_use_scratch(B, N, m, sorted_copy, monkeypatch):
    """Clouds beyond the on-chip capacity: running minimum in global scratch, with the sorted
    copy and chunk skipping (20 bytes per point) or without (4 bytes per point)."""
    data.use_paths(monkeypatch, "fps_unsorted" if sorted_copy == "0" else None)
    assert _lib.lib().tpk_fps_scratch_bytes(B, N, m) == B * N * (20 if sorted_copy == "1" else 4)
    x = data.gaussian_mixture(B, N, seed=5000 + N)
    got = npy(tpk.furthest_point_sample(cu(x), m))
    np.testing.assert_array_equal(got, orc.fps(x, m))
    assert _lib.device_status() == 0


@pytest.mark.parametrize("n", [3, 37, 700, 5000, 20000])
@pytest.mark.parametrize("sorted_copy", ["1", "0"])
def test_fps_scratch_kernel_tie_break_and_skip_rule(n, sorted_copy, monkeypatch):
    data.use_paths(monkeypatch, "fps_global", "fps_unsorted" if sorted_copy == "0" else None)
    rng = np.random.default_rng(n)
    pts = np.zeros((2, n, 3), np.float32)
    pts[:, 0] = (1.0, 1.0, 1.0)
    pts[:, 1:] = (1.0, 1.0, 1.5)
    far = rng.choice(np.arange(1, n), size=max(1, (n - 1) // 2), replace=False)
    pts[0, far] = (5.0, 1.0, 1.0)
    pts[1, 1:] = rng.integers(0, 3, size=(n - 1, 3)).astype(np.float32)
    m = min(n, 12)
    np.testing.assert_array_equal(npy(tpk.furthest_point_sample(cu(pts), m)), orc.fps(pts, m))
    x = data.unit_ball(2, n, seed=n)
    mm = min(n, 200)
    np.testing.assert_array_equal(npy(tpk.furthest_point_sample(cu(x), mm)), orc.fps(x, mm))


@pytest.mark.parametrize("B,N,m,env", [(3, 1000, 200, None), (2, 16384, 700, None), (2, 16384, 700, "fps_unsorted"),
                                       (1, 150000, 40, None), (1, 150000, 40, "fps_unsorted"), (4, 257, 257, None)])
def test_fps_returns_sampled_coordinates(B, N, m, env, monkeypatch):
    """return_xyz: the coordinates of the samples (behind every kernel variant)."""
    data.use_paths(monkeypatch, env)
    x = cu(data.unit_ball(B, N, seed=2100 + N))
    idx, centres = tpk.furthest_point_sample(x, m, return_xyz=True)
    np.testing.assert_array_equal(npy(idx), npy(tpk.furthest_point_sample(x, m)))
    want = torch.gather(x, 1, idx.long().unsqueeze(-1).expand(-1, -1, 3))
    same_bits(npy(centres), npy(want))
    # no candidate at all: every sample is point 0
    tiny = cu(np.full((2, 40, 3), 0.001, np.float32))
    idx, centres = tpk.furthest_point_sample(tiny, 7, return_xyz=True)
    assert (npy(idx) == 0).all() and (npy(centres) == np.float32(0.001)).all()


@pytest.mark.parametrize("kind", ["two_blobs", "duplicates", "line", "shell"])
@pytest.mark.parametrize("cfg", [None, "8:128:4", "2:512:8", "1:128:32", "16:64:4", "1:512:8"])
def test_fps_several_samples_per_exchange_hard_cases(kind, cfg, monkeypatch):
    """The batched kernel accepts a candidate only when it is provably the next sample: clouds
    where the largest minima sit next to each other (two tight blobs, a line), where many points
    coincide (equal keys everywhere) and a thin shell, through several cluster shapes."""
    rng = np.random.default_rng(len(kind))
    B, n, m = 3, 3000, 1200
    if kind == "two_blobs":
        x = (rng.standard_normal((B, n, 3)) * 0.01 + (rng.integers(0, 2, (B, n, 1)) * 3.0)).astype(np.float32)
    elif kind == "duplicates":
        base = rng.uniform(-1, 1, (B, 40, 3)).astype(np.float32)
        x = np.take_along_axis(base, rng.integers(0, 40, (B, n, 1)).repeat(3, 2), 1)
    elif kind == "line":
        x = np.zeros((B, n, 3), np.float32)
        x[..., 0] = rng.uniform(0.1, 5, (B, n))
    else:
        d = rng.standard_normal((B, n, 3))
        x = (d / np.linalg.norm(d, axis=2, keepdims=True) * (1 + 1e-4 * rng.standard_normal((B, n, 1)))).astype(np.float32)
    want = orc.fps(x, m)
    data.use_paths(monkeypatch, "fps_sorted", cfg and "fps_config=" + cfg)
    np.testing.assert_array_equal(npy(tpk.furthest_point_sample(cu(x), m)), want)
    assert _lib.device_status() == 0


def test_fps_all_points_skipped():
    tiny = np.full((2, 40, 3), 0.001, np.float32)
    assert npy(tpk.furthest_point_sample(cu(tiny), 7)).tolist() == [[0] * 7] * 2


# ------------------------------------------------------------------------ ball query

def test_ball_query_known_answers(known_answers):
    ka = known_answers["ball_query_dense_cuda"]
    idx, dist = tpk.ball_query(ka["radius"], ka["nsample"], cu(np.asarray(ka["x"], np.float32)),
                               cu(np.asarray(ka["y"], np.float32)))
    assert idx.dtype == torch.int64 and npy(idx).tolist() == ka["idx"]
    np.testing.assert_allclose(npy(dist), np.asarray(ka["dist"], np.float32), atol=1e-6)
    for name in ("ball_query_partial_cuda", "ball_query_partial_cpu"):
        ka = known_answers[name]
        idx, dist = tpk.ball_query(ka["radius"], ka["nsample"], cu(np.asarray(ka["x"], np.float32)),
                                   cu(np.asarray(ka["y"], np.float32)), mode="PARTIAL_DENSE",
                                   batch_x=cu(np.asarray(ka["batch_x"])), batch_y=cu(np.asarray(ka["batch_y"])))
        assert npy(idx).tolist() == ka["idx"]
        np.testing.assert_allclose(npy(dist), np.asarray(ka["dist"], np.float32), atol=1e-6)


@pytest.mark.parametrize("B,N,M,r,ns", [(4, 4096, 1024, 0.2, 32), (2, 1025, 77, 0.1, 32), (3, 5, 9, 0.5, 4),
                                        (2, 1, 3, 10.0, 3), (2, 3000, 300, 0.8, 32), (1, 2048, 2048, 0.05, 1),
                                        (2, 1500, 40, 1e-4, 16), (16, 1024, 256, 0.4, 32)])
def test_ball_query_dense_matches_oracle(B, N, M, r, ns):
    x = data.unit_ball(B, N, seed=N + M)
    y = x[:, torch.randperm(N, generator=data.gen(N))[: min(M, N)]].contiguous() if M <= N else data.unit_ball(B, M, seed=5)
    idx, dist = tpk.ball_query(r, ns, cu(x), cu(y), mode="dense")
    oi, od = orc.ball_query_dense(r, ns, x, y)
    np.testing.assert_array_equal(npy(idx), oi)
    same_bits(npy(dist), od)


@pytest.mark.parametrize("case", ["uniform", "blobs", "offset", "flat", "far_queries", "ns1", "ns100"])
def test_ball_query_dense_grid_path_matches_oracle(case, monkeypatch):
    """Clouds large enough for the uniform-grid search: same bits as the oracle (and as the scan),
    including centres handed back to the scan (dense blobs) and degenerate grids."""
    g = data.gen(hash(case) % 1000)
    B, N, M, r, ns = 3, 9000, 700, 0.07, 32
    if case == "blobs":
        x = data.gaussian_mixture(B, N, seed=11, comps=6)
        r = 0.05
    else:
        x = data.unit_ball(B, N, seed=12)
    if case == "offset":
        x = (x + torch.tensor([1000.0, -500.0, 250.0])).contiguous()
    if case == "flat":
        x[..., 2] = 0.25
    y = x[:, torch.randperm(N, generator=g)[:M]].contiguous()
    if case == "far_queries":
        y = (y + 3.0).contiguous()
        y[:, :50] = x[:, :50]
    if case == "ns1":
        ns = 1
    if case == "ns100":
        ns, r = 100, 0.2
    assert _lib.lib().tpk_ball_query_dense_scratch_bytes(B, N, M, ns) > 0
    oi, od = orc.ball_query_dense(r, ns, x, y)
    # the grid in shared memory (where it fits), the grid in global memory, the plain scan
    for env in (None, "ball_query_global_grid", "ball_query_scan"):
        data.use_paths(monkeypatch, env)
        idx, dist = tpk.ball_query(r, ns, cu(x), cu(y), mode="dense")
        np.testing.assert_array_equal(npy(idx), oi)
        same_bits(npy(dist), od)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("case", ["crowded_layer", "nonfinite_centres", "nonfinite_points", "thin_cells", "many_centres"])
def test_ball_query_dense_shared_memory_grid_edge_cases(case):
    """The shared-memory grid hands back what it cannot answer: a layer with more points than
    fit, centres without a cell, clouds without a grid; cells exactly one radius wide; more
    centres than one list pass takes."""
    B, N, M, r, ns = 2, 6000, 500, 0.08, 16
    x = data.unit_ball(B, N, seed=31).numpy().copy()
    if case == "crowded_layer":
        x[0, :5000, 2] = 0.123  # one z layer holds most of cloud 0
    if case == "thin_cells":
        r = 0.3  # the radius, not the cell budget, sets the cell size
    if case == "many_centres":
        M = 5000
    y = np.array(x[:, :M])
    if case == "nonfinite_centres":
        y[0, 3, 1] = np.nan
        y[1, 7, 2] = np.inf
    if case == "nonfinite_points":
        x[1, 10, 0] = np.inf
    assert _lib.lib().tpk_ball_query_dense_scratch_bytes(B, N, M, ns) == (B * M + 255) // 256 * 256
    idx, dist = tpk.ball_query(r, ns, cu(x), cu(y), mode="dense")
    oi, od = orc.ball_query_dense(r, ns, x, y)
    np.testing.assert_array_equal(npy(idx), oi)
    same_bits(npy(dist), od)


@pytest.mark.parametrize("kind", ["ball", "mixture"])
def test_ball_query_dense_huge_clouds_use_the_hashed_grid(kind, monkeypatch):
    """Clouds of 2^18+ points: the hashed grid in global scratch, against the oracle, the older
    bounding-box grid and the scan (crowded centres of the mixture go back to the scan)."""
    B, N, M, r, ns = 2, 270000, 400, 0.03, 32
    x = data.unit_ball(B, N, seed=41) if kind == "ball" else data.gaussian_mixture(B, N, seed=42, comps=8)
    y = x[:, torch.randperm(N, generator=data.gen(43))[:M]].contiguous()
    need = _lib.lib().tpk_ball_query_dense_scratch_bytes(B, N, M, ns)
    assert need > B * N * 20
    oi, od = orc.ball_query_dense(r, ns, x, y)
    for env in (None, "ball_query_global_grid", "ball_query_scan"):
        data.use_paths(monkeypatch, env)
        idx, dist = tpk.ball_query(r, ns, cu(x), cu(y), mode="dense")
        np.testing.assert_array_equal(npy(idx), oi)
        same_bits(npy(dist), od)


def test_ball_query_dense_boundary_is_strict_partial_is_inclusive():
    x = np.array([[[0, 0, 0], [0.5, 0, 0], [0.25, 0, 0]]], np.float32)
    y = np.array([[[0, 0, 0]]], np.float32)
    idx, dist = tpk.ball_query(0.5, 3, cu(x), cu(y))
    assert npy(idx).tolist() == [[[0, 2, 0]]] and npy(dist).tolist() == [[[0.0, 0.0625, -1.0]]]
    b = torch.zeros(3, dtype=torch.long)
    idx, dist = tpk.ball_query(0.5, 3, cu(x[0]), cu(y[0]), mode="partial_dense", batch_x=cu(b), batch_y=cu(b[:1]))
    assert npy(idx).tolist() == [[0, 1, 2]] and npy(dist).tolist() == [[0.0, 0.25, 0.0625]]


def test_ball_query_partial_golden_and_oracle(golden_dir):
    p = np.load(os.path.join(golden_dir, "partial.npz"))
    r, ns = float(p["radius"]), int(p["nsample"])
    idx, d2 = tpk.ball_query(r, ns, cu(p["x"]), cu(p["y"]), mode="partial_dense",
                             batch_x=cu(p["batch_x"]), batch_y=cu(p["batch_y"]))
    oi, od = orc.ball_query_partial(r, ns, p["x"], p["y"], p["batch_x"], p["batch_y"])
    np.testing.assert_array_equal(npy(idx), oi)
    same_bits(npy(d2), od)
    r2 = np.float32(r) * np.float32(r)
    for q in range(oi.shape[0]):  # the reference CPU result as a set (strict radius there)
        got = {int(i) for i, d in zip(npy(idx)[q], npy(d2)[q]) if d >= 0 and d != r2}
        assert got == {int(i) for i, d in zip(p["idx"][q], p["d2"][q]) if d >= 0}


@pytest.mark.parametrize("seed,ns", [(1, 16), (2, 64), (3, 1)])
def test_ball_query_partial_ragged_segments(seed, ns):
    g = data.gen(seed)
    sizes = [1, 700, 3, 0, 1500, 2, 260, 1100]       # id 3 has no support points
    qsizes = [1, 90, 0, 4, 333, 2, 0, 270]           # ids 2 and 6 have no queries
    x = torch.cat([torch.rand(s, 3, generator=g) for s in sizes])
    bx = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(sizes)])
    y = torch.cat([torch.rand(s, 3, generator=g) for s in qsizes])
    by = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(qsizes)])
    idx, d2 = tpk.ball_query(0.12, ns, cu(x), cu(y), mode="partial_dense", batch_x=cu(bx), batch_y=cu(by))
    oi, od = orc.ball_query_partial(0.12, ns, x, y, bx, by)
    np.testing.assert_array_equal(npy(idx), oi)
    same_bits(npy(d2), od)


def test_ball_query_partial_scene_scale():
    x, y, bx, by = data.packed_planes(n_scenes=5, lo=2000, hi=9000, seed=3001)
    idx, d2 = tpk.ball_query(0.05, 64, cu(x), cu(y), mode="partial_dense", batch_x=cu(bx), batch_y=cu(by))
    oi, od = orc.ball_query_partial(0.05, 64, x, y, bx, by)
    np.testing.assert_array_equal(npy(idx), oi)
    same_bits(npy(d2), od)


@pytest.mark.parametrize("case", ["scenes", "crowded", "overlapping_segments", "nonfinite", "far_offsets", "ns1"])
def test_ball_query_partial_hash_grid_matches_oracle_and_scan(case, monkeypatch):
    """4096+ packed points go through the hashed grid: same indices and distance bits as the
    oracle and as the scan of the segments, also for queries the grid hands back (crowded
    neighbourhoods, non-finite coordinates, coordinates so large that a cell is thinner than their rounding)."""
    rng = np.random.default_rng(len(case))
    r, ns = 0.05, 64
    if case == "scenes":
        x, y, bx, by = data.packed_planes(n_scenes=6, lo=3000, hi=12000, seed=3002)
    elif case == "crowded":
        # hundreds of points inside one ball: more hits than the buffer takes
        sizes, qsizes = [5000, 3000], [400, 300]
        x = torch.from_numpy(np.concatenate([rng.normal(0, 0.03, (s, 3)) for s in sizes]).astype(np.float32))
        y = torch.from_numpy(np.concatenate([rng.normal(0, 0.03, (s, 3)) for s in qsizes]).astype(np.float32))
        bx = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(sizes)])
        by = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(qsizes)])
    else:
        # every segment fills the same unit cube: neighbours must come from the query's own segment only
        sizes, qsizes = [3000, 1, 4000, 0, 2500], [200, 3, 300, 5, 0]
        x = torch.from_numpy(rng.uniform(0, 1, (sum(sizes), 3)).astype(np.float32))
        y = torch.from_numpy(rng.uniform(0, 1, (sum(qsizes), 3)).astype(np.float32))
        bx = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(sizes)])
        by = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(qsizes)])
        r = 0.08
        if case == "nonfinite":
            x[17, 0] = float("inf")
            x[5000, 2] = float("nan")
            y[3, 1] = float("nan")
            y[250, 0] = float("-inf")
        if case == "far_offsets":
            x = x + 30000.0
            y = y + 30000.0
        if case == "ns1":
            ns = 1
    assert _lib.lib().tpk_ball_query_partial_dense_scratch_bytes(x.shape[0], y.shape[0], r) > 0
    oi, od = orc.ball_query_partial(r, ns, x, y, bx, by)
    for env in (None, "ball_query_scan"):
        data.use_paths(monkeypatch, env)
        idx, d2 = tpk.ball_query(r, ns, cu(x), cu(y), mode="partial_dense", batch_x=cu(bx), batch_y=cu(by))
        np.testing.assert_array_equal(npy(idx), oi)
        same_bits(npy(d2), od)


# ------------------------------------------------------------------ three_nn and kNN

@pytest.mark.parametrize("B,n,m", [(4, 4096, 1024), (2, 1000, 2000), (3, 77, 3), (2, 10, 2), (2, 5, 1), (16, 256, 64),
                                   (2, 3000, 10000), (3, 700, 256), (1, 100000, 300)])
def test_three_nn_matches_oracle(B, n, m):
    unknown = data.unit_ball(B, n, seed=n)
    known = data.unit_ball(B, m, seed=m + 1)
    dist, idx = tpk.three_nn(cu(unknown), cu(known))
    od2, oi = orc.three_nn(unknown, known)
    assert idx.dtype == torch.int32
    np.testing.assert_array_equal(npy(idx), oi)
    with np.errstate(invalid="ignore"):
        same_bits(npy(dist), np.sqrt(od2))


def test_three_nn_duplicates_keep_lowest_index_first():
    known = np.zeros((1, 6, 3), np.float32)
    known[0, :, 0] = [1, 1, 1, 2, 1, 0.5]
    unknown = np.zeros((1, 3, 3), np.float32)
    dist, idx = tpk.three_nn(cu(unknown), cu(known))
    assert npy(idx)[0, 0].tolist() == [5, 0, 1]
    od2, oi = orc.three_nn(unknown, known)
    np.testing.assert_array_equal(npy(idx), oi)


def _three_nn_grid_cases():
    rng = np.random.default_rng(77)
    cases = {}
    cases["uniform"] = (data.unit_ball(3, 6000, seed=11), data.unit_ball(3, 8192, seed=12))
    # queries far outside the bounding box of the known points, and on its faces
    u = data.unit_ball(2, 3000, seed=13) * 4.0
    u[:, :50] = 1.0
    cases["outside"] = (u, data.unit_ball(2, 4096, seed=14))
    # clustered known points: most cells empty, a few crowded; many exact duplicates
    k = (rng.standard_normal((2, 5000, 3)) * 0.01 + rng.integers(0, 3, (2, 5000, 1))).astype(np.float32)
    k[:, 1000:1600] = k[:, :600]
    cases["clustered_duplicates"] = (rng.uniform(-1, 4, (2, 2500, 3)).astype(np.float32), k)
    # known points on a plane (one grid dimension collapses) and on a coarse lattice (ties)
    k = rng.uniform(0, 1, (2, 4500, 3)).astype(np.float32)
    k[..., 2] = 0.25
    cases["planar"] = (rng.uniform(0, 1, (2, 2000, 3)).astype(np.float32), k)
    k = rng.integers(0, 12, (1, 6000, 3)).astype(np.float32) / 4
    cases["lattice_ties"] = (rng.integers(0, 24, (1, 3000, 3)).astype(np.float32) / 8, k)
    # the PointNet++ shape: upsampling 4096 -> 16384
    x = data.unit_ball(2, 16384, seed=15)
    cases["upsample"] = (x, np.ascontiguousarray(x[:, ::4]))
    # more than 8192 known points: the grid is staged by layers; sparse regions and far
    # queries need rings beyond the staged layers and go to the scan
    cases["many_known"] = (data.unit_ball(2, 5000, seed=16) * 1.2, data.unit_ball(2, 12000, seed=17))
    k = (rng.standard_normal((2, 11000, 3)) * 0.05 + rng.integers(0, 3, (2, 11000, 1))).astype(np.float32)
    cases["many_known_clustered"] = (rng.uniform(-1, 3, (2, 3000, 3)).astype(np.float32), k)
    return cases


@pytest.mark.parametrize("name", ["uniform", "outside", "clustered_duplicates", "planar", "lattice_ties", "upsample",
                                  "many_known", "many_known_clustered"])
def test_three_nn_grid_path_matches_oracle(name, monkeypatch):
    unknown, known = _three_nn_grid_cases()[name]
    b, n, m = unknown.shape[0], unknown.shape[1], known.shape[1]
    assert _lib.lib().tpk_three_nn_scratch_bytes(b, n, m) > 0  # the grid path is the one tested
    od2, oi = orc.three_nn(unknown, known)
    # the grid in shared memory (up to 8192 known points), then the grid in global memory
    for env in (None, "three_nn_global_grid", "three_nn_scan"):
        data.use_paths(monkeypatch, env)
        dist, idx = tpk.three_nn(cu(unknown), cu(known))
        np.testing.assert_array_equal(npy(idx), oi)
        same_bits(npy(dist), np.sqrt(od2))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("env", [None, "three_nn_global_grid"])
def test_three_nn_grid_path_nonfinite_falls_back_to_scan(env, monkeypatch):
    data.use_paths(monkeypatch, env)
    unknown = data.unit_ball(2, 1500, seed=21).numpy().copy()
    known = data.unit_ball(2, 4096, seed=22).numpy().copy()
    unknown[0, 7, 1] = np.inf
    unknown[1, 9, 0] = np.nan
    known[1, 100, 2] = np.inf  # cloud 1: no grid at all
    dist, idx = tpk.three_nn(cu(unknown), cu(known))
    od2, oi = orc.three_nn(unknown, known)
    np.testing.assert_array_equal(npy(idx), oi)
    with np.errstate(invalid="ignore"):
        same_bits(npy(dist), np.sqrt(od2))


def test_knn_known_answer(known_answers):
    ka = known_answers["knn"]
    s, q = cu(np.asarray(ka["support"], np.float32)), cu(np.asarray(ka["query"], np.float32))
    idx, d2 = tpk.knn(s, q, 3)
    assert idx.dtype == torch.int64 and npy(idx).tolist() == ka["k3_idx"]
    assert npy(d2).tolist() == ka["k3_dist"]
    assert npy(tpk.knn(s, q, 2)[0]).tolist() == ka["k2_idx"]
    with pytest.raises(RuntimeError):
        tpk.knn(s, q, ka["k_too_large"])


def test_knn_golden_bit_exact(golden_dir):
    p = np.load(os.path.join(golden_dir, "plumbing.npz"))
    for k in (3, 16):
        idx, d2 = tpk.knn(cu(p["x"]), cu(p["y"]), k)
        np.testing.assert_array_equal(npy(idx), p["knn%d_idx" % k])
        same_bits(npy(d2), p["knn%d_d2" % k])


@pytest.mark.parametrize("B,N,M,k", [(4, 4096, 1024, 3), (2, 3000, 500, 16), (2, 700, 130, 1), (1, 2500, 300, 64),
                                     (3, 40, 17, 40), (16, 1500, 64, 8)])
def test_knn_dense_matches_oracle(B, N, M, k):
    s = data.unit_ball(B, N, seed=N + k)
    q = data.unit_ball(B, M, seed=M + k)
    idx, d2 = tpk.knn(cu(s), cu(q), k)
    oi, od = orc.knn(s, q, k)
    np.testing.assert_array_equal(npy(idx), oi)
    same_bits(npy(d2), od)


def test_knn_partial_matches_per_segment_dense():
    x, y, bx, by = data.packed_planes(n_scenes=4, lo=1500, hi=5000, seed=3002)
    # a short segment (fewer support points than k) and one without queries
    x = torch.cat([x, torch.rand(5, 3)]); bx = torch.cat([bx, torch.full((5,), 4)])
    y = torch.cat([y, torch.rand(2, 3)]); by = torch.cat([by, torch.full((2,), 4)])
    x = torch.cat([x, torch.rand(30, 3)]); bx = torch.cat([bx, torch.full((30,), 6)])
    idx, d2 = tpk.knn(cu(x), cu(y), 16, batch_support=cu(bx), batch_pos=cu(by))
    oi, od = orc.knn_segmented(x, y, bx, by, 16)
    np.testing.assert_array_equal(npy(idx), oi)
    same_bits(npy(d2), od)


@pytest.mark.parametrize("B,N,M,k", [(2, 20000, 3000, 16), (1, 6000, 6000, 3), (3, 5000, 700, 64), (2, 9000, 100, 33),
                                     (1, 50000, 2000, 1)])
@pytest.mark.parametrize("kind", ["ball", "planes", "clustered"])
def test_knn_dense_grid_matches_scan_and_oracle(B, N, M, k, kind, monkeypatch):
    """Clouds large enough for the hashed grid: its answers (and the scan's behind it) against the
    oracle, and grid against scan bit for bit.  Uniform, planar (the density estimate is
    volumetric) and clustered clouds with queries far from every point."""
    g = data.gen(N + k)
    if kind == "ball":
        s, q = data.unit_ball(B, N, seed=N + k), data.unit_ball(B, M, seed=M + k)
    elif kind == "planes":
        s = torch.rand(B, N, 3, generator=g) * 5
        s[..., 2] = torch.randint(0, 3, (B, N), generator=g).float() + 0.01 * torch.randn(B, N, generator=g)
        q = s[:, torch.randperm(N, generator=g)[:M]].contiguous() + 0.001
    else:
        s = 0.02 * torch.randn(B, N, 3, generator=g) + torch.randint(0, 3, (B, N, 1), generator=g) * 4.0
        q = torch.rand(B, M, 3, generator=g) * 10 - 1   # most queries sit in empty space
    assert _lib.lib().tpk_knn_dense_scratch_bytes(B, N, M, k) > 0
    idx, d2 = tpk.knn(cu(s), cu(q), k)
    data.use_paths(monkeypatch, "knn_scan")
    assert _lib.lib().tpk_knn_dense_scratch_bytes(B, N, M, k) == 0
    sidx, sd2 = tpk.knn(cu(s), cu(q), k)
    np.testing.assert_array_equal(npy(idx), npy(sidx))
    same_bits(npy(d2), npy(sd2))
    if N * M * B <= 150_000_000:
        oi, od = orc.knn(s, q, k)
        np.testing.assert_array_equal(npy(idx), oi)
        same_bits(npy(d2), od)


def test_knn_grid_ties_and_nonfinite(monkeypatch):
    """Exact distance ties (lattice points: index order among equals) and coordinates that are
    not finite go through the grid and its fallback with the scan's results."""
    g = data.gen(3)
    s = torch.randint(0, 12, (2, 5000, 3), generator=g).float() * 0.25
    q = torch.randint(0, 12, (2, 400, 3), generator=g).float() * 0.25 + 0.125
    s[0, 17, 0] = float("inf")
    s[1, 9, 2] = float("nan")
    q[0, 3, 1] = float("nan")
    q[1, 5, 0] = float("-inf")
    idx, d2 = tpk.knn(cu(s), cu(q), 8)
    data.use_paths(monkeypatch, "knn_scan")
    sidx, sd2 = tpk.knn(cu(s), cu(q), 8)
    np.testing.assert_array_equal(npy(idx), npy(sidx))
    same_bits(npy(d2), npy(sd2))


@pytest.mark.parametrize("k", [16, 40])
def test_knn_partial_grid_matches_scan_and_oracle(k, monkeypatch):
    x, y, bx, by = data.packed_planes(n_scenes=5, lo=3000, hi=9000, seed=3005)
    # a short segment (fewer support points than k), one without queries, one far away
    x = torch.cat([x, torch.rand(5, 3)]); bx = torch.cat([bx, torch.full((5,), 5)])
    y = torch.cat([y, torch.rand(2, 3)]); by = torch.cat([by, torch.full((2,), 5)])
    x = torch.cat([x, torch.rand(30, 3)]); bx = torch.cat([bx, torch.full((30,), 7)])
    x = torch.cat([x, torch.rand(3000, 3) + 50]); bx = torch.cat([bx, torch.full((3000,), 8)])
    y = torch.cat([y, torch.rand(40, 3) + 50]); by = torch.cat([by, torch.full((40,), 8)])
    assert _lib.lib().tpk_knn_partial_dense_scratch_bytes(x.shape[0], y.shape[0], k) > 0
    idx, d2 = tpk.knn(cu(x), cu(y), k, batch_support=cu(bx), batch_pos=cu(by))
    oi, od = orc.knn_segmented(x, y, bx, by, k)
    np.testing.assert_array_equal(npy(idx), oi)
    same_bits(npy(d2), od)
    data.use_paths(monkeypatch, "knn_scan")
    sidx, sd2 = tpk.knn(cu(x), cu(y), k, batch_support=cu(bx), batch_pos=cu(by))
    np.testing.assert_array_equal(npy(idx), npy(sidx))
    same_bits(npy(d2), npy(sd2))


# --------------------------------------------------------- interpolation and grouping

@pytest.mark.parametrize("B,C,m,n", [(4, 64, 1024, 4096), (2, 7, 33, 1001), (3, 30, 100, 500), (2, 130, 64, 256)])
def test_three_interpolate_forward_backward(B, C, m, n):
    g = data.gen(n)
    known = torch.rand(B, m, 3, generator=g)
    unknown = torch.rand(B, n, 3, generator=g)
    feat = torch.randn(B, C, m, generator=g)
    od2, oi = orc.three_nn(unknown, known)
    dist = torch.from_numpy(np.sqrt(od2))
    w = 1.0 / (dist + 1e-8)
    w = (w / w.sum(2, keepdim=True)).contiguous()
    f = cu(feat).requires_grad_(True)
    out = tpk.three_interpolate(f, cu(oi), cu(w))
    want = orc.three_interpolate(feat, oi, w)
    np.testing.assert_allclose(npy(out), want, rtol=1e-5, atol=1e-6)
    gout = torch.randn(out.shape, generator=g)
    out.backward(cu(gout))
    np.testing.assert_allclose(npy(f.grad), orc.three_interpolate_grad(gout, oi, w, m), rtol=1e-4, atol=1e-4)


def test_three_interpolate_golden(golden_dir):
    p = np.load(os.path.join(golden_dir, "plumbing.npz"))
    f = cu(p["feat"]).requires_grad_(True)
    out = tpk.three_interpolate(f, cu(p["nn_idx"].astype(np.int32)), cu(p["weight"]))
    np.testing.assert_allclose(npy(out), p["interp"], rtol=1e-5, atol=1e-6)
    out.backward(cu(p["interp_gout"]))
    np.testing.assert_allclose(npy(f.grad), p["interp_grad"], rtol=1e-4, atol=1e-4)


def test_grouping_known_answer(known_answers):
    ka = known_answers["grouping"]
    out = tpk.grouping_operation(cu(np.asarray(ka["features"], np.float32)), cu(np.asarray(ka["idx"], np.int64)))
    np.testing.assert_array_equal(npy(out), np.asarray(ka["expected"], np.float32))


@pytest.mark.parametrize("B,C,N,P,S", [(4, 64, 4096, 1024, 32), (2, 5, 100, 33, 3), (3, 130, 257, 64, 32),
                                       (1, 3, 60000, 500, 16), (2, 17, 1000, 1, 1)])
def test_grouping_forward_backward(B, C, N, P, S, monkeypatch):
    g = data.gen(N + P)
    feat = torch.randn(B, C, N, generator=g)
    idx = torch.randint(0, N, (B, P, S), generator=g)
    f = cu(feat).requires_grad_(True)
    out = tpk.grouping_operation(f, cu(idx))
    np.testing.assert_array_equal(npy(out), orc.grouping(feat, idx))
    gout = torch.randn(out.shape, generator=g)
    out.backward(cu(gout))
    want = orc.grouping_grad(gout, idx, N)
    np.testing.assert_allclose(npy(f.grad), want, rtol=1e-4, atol=1e-4)
    # the shared-memory-atomics kernels and the global-atomics fallback give the same sums
    for path in ("scatter_atomic", "scatter_global"):
        data.use_paths(monkeypatch, path)
        f2 = cu(feat).requires_grad_(True)
        tpk.grouping_operation(f2, cu(idx)).backward(cu(gout))
        np.testing.assert_allclose(npy(f2.grad), want, rtol=1e-4, atol=1e-4)


def test_rows_of_exactly_48_kb_in_a_fresh_process():
    """Three rows of 4096 floats are exactly the 48 KB a launch may take without raising the
    kernel's shared-memory limit - but the kernel's static mbarrier counts too.  In a process
    that has not run the same kernel on longer rows before, the call must still work."""
    import subprocess
    import sys
    code = (
        "import torch, torch_points_kernels_b200 as tpk\n"
        "g = torch.Generator().manual_seed(5)\n"
        "f = torch.randn(2, 3, 4096, generator=g).cuda(); idx = torch.randint(0, 4096, (2, 1024, 32), generator=g).cuda()\n"
        "out = tpk.grouping_operation(f, idx)\n"
        "ref = torch.gather(f, 2, idx.view(2, 1, -1).expand(2, 3, -1)).view(2, 3, 1024, 32)\n"
        "assert torch.equal(out, ref)\n"
        "p = torch.randn(2, 3, 4096, generator=g).cuda(); i3 = torch.randint(0, 4096, (2, 9000, 3), generator=g).int().cuda()\n"
        "w = torch.rand(2, 9000, 3, generator=g).cuda()\n"
        "up = tpk.three_interpolate(p, i3, w)\n"
        "want = (torch.gather(p, 2, i3.long().view(2, 1, -1).expand(2, 3, -1)).view(2, 3, 9000, 3) * w.unsqueeze(1)).sum(-1)\n"
        "assert torch.allclose(up, want, rtol=1e-5, atol=1e-5)\n"
        "print('ok')\n")
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    r = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


@pytest.mark.parametrize("B,C,N,P,S,kind", [
    (2, 64, 16384, 4096, 32, "ball"),      # level-1 shape: eight tiles of 16384 positions
    (2, 5, 9000, 1000, 32, "ball"),        # two tiles, the second one short
    (1, 3, 12000, 700, 24, "one"),         # every position adds to the same column: runs longer than a chunk
    (2, 4, 9000, 600, 30, "sorted"),       # targets already in order
    (1, 2, 10000, 333, 7, "random"),       # positions not a multiple of four: tiles staged by hand
    (1, 1, 40000, 5000, 8, "random"),      # a row that fills most of shared memory: shorter tiles
])
def test_grouping_backward_sorted_path(B, C, N, P, S, kind):
    """The gradient through the inverted index (tpk_grouping_grad_ws) against the fp64 sums of the
    oracle, on index patterns that stress its runs: ball-query padding, one target, sorted targets."""
    g = data.gen(N + P + S)
    if kind == "ball":
        idx = torch.randint(0, N, (B, P, S), generator=g)
        cnt = torch.randint(1, S + 1, (B, P, 1), generator=g)
        slot = torch.arange(S).view(1, 1, S)
        idx = torch.where(slot < cnt, idx, idx[:, :, :1])  # unused slots repeat the first index
    elif kind == "one":
        idx = torch.full((B, P, S), 77, dtype=torch.long)
    elif kind == "sorted":
        idx = torch.sort(torch.randint(0, N, (B, P * S), generator=g), dim=1).values.view(B, P, S)
    else:
        idx = torch.randint(0, N, (B, P, S), generator=g)
    gout = torch.randn(B, C, P, S, generator=g)
    assert _lib.lib().tpk_grouping_grad_scratch_bytes(B, C, N, P, S) > 0
    got = tpk.torchpoints.grouping_backward(cu(gout), cu(idx), N)
    want = orc.grouping_grad(gout, idx, N)
    tol = 1e-4 * max(1.0, float(np.abs(want).max()))
    np.testing.assert_allclose(npy(got), want, rtol=1e-4, atol=tol)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("B,N,M,C,r", [(2, 16384, 4096, 64, 0.1), (3, 4096, 1024, 7, 0.2), (2, 500, 100, 130, 0.4),
                                       (1, 70000, 64, 3, 0.05), (2, 1024, 256, 0, 0.3)])
def test_fused_sa_group_equals_the_unfused_sequence(B, N, M, C, r):
    """tpk.sa_group against gather + ball_query + two grouping_operations + subtraction + cat,
    bit for bit, forward; the gradient of the features against grouping's backward."""
    x = cu(data.unit_ball(B, N, seed=N + C))
    g = data.gen(N)
    feat = cu(torch.randn(B, C, N, generator=g)).requires_grad_(True) if C else None
    fps = tpk.furthest_point_sample(x, M)
    new_xyz, idx, out = tpk.sa_group(x, feat, fps, r, 32)
    want_xyz = torch.gather(x, 1, fps.long().unsqueeze(-1).expand(-1, -1, 3)).contiguous()
    want_idx, _ = tpk.ball_query(r, 32, x, want_xyz, mode="dense")
    rel = tpk.grouping_operation(x.transpose(1, 2).contiguous(), want_idx) - want_xyz.transpose(1, 2).unsqueeze(-1)
    same_bits(npy(new_xyz), npy(want_xyz))
    np.testing.assert_array_equal(npy(idx), npy(want_idx))
    if C:
        f2 = feat.detach().clone().requires_grad_(True)
        want = torch.cat([rel, tpk.grouping_operation(f2, want_idx)], dim=1)
        same_bits(npy(out), npy(want))
        gout = cu(torch.randn(out.shape, generator=g))
        out.backward(gout)
        want.backward(gout)
        np.testing.assert_allclose(npy(feat.grad), npy(f2.grad), rtol=1e-4, atol=1e-4)
    else:
        same_bits(npy(out), npy(rel))
    assert _lib.device_status() == 0


def test_grouping_golden(golden_dir):
    p = np.load(os.path.join(golden_dir, "plumbing.npz"))
    f = cu(p["gfeat"]).requires_grad_(True)
    out = tpk.grouping_operation(f, cu(p["gidx"]))
    np.testing.assert_array_equal(npy(out), p["grouped"])
    out.backward(cu(p["grouped_gout"]))
    np.testing.assert_allclose(npy(f.grad), p["grouped_grad"], rtol=1e-4, atol=1e-4)


# ------------------------------------------------------------------------- chamfer

def test_chamfer_known_answers(known_answers):
    ka = known_answers["chamfer"]
    x1, x2 = cu(np.asarray(ka["xyz1"], np.float32)), cu(np.asarray(ka["xyz2"], np.float32))
    assert abs(cd.chamfer_dist(x1, x2).item() - ka["dist"]) < 10 ** -ka["places"]
    assert abs(cd.chamfer_dist(x1, x2, True).item() - ka["dist_ignore_zeros"]) < 10 ** -ka["places"]


@pytest.mark.parametrize("B,n,m", [(4, 2048, 2048), (2, 1000, 1777), (3, 5, 1), (64, 300, 200)])
def test_chamfer_forward_backward(B, n, m):
    c1, c2 = data.chamfer_pair(B, max(n, m), seed=4000 + n)
    c1, c2 = c1[:, :n].contiguous(), c2[:, :m].contiguous()
    x1, x2 = cu(c1).requires_grad_(True), cu(c2).requires_grad_(True)
    d1, d2 = cd.ChamferFunction.apply(x1, x2)
    o1, o2, i1, i2 = orc.chamfer(c1, c2)
    same_bits(npy(d1), o1)
    same_bits(npy(d2), o2)
    g = data.gen(n)
    g1, g2 = torch.randn(B, n, generator=g), torch.randn(B, m, generator=g)
    torch.autograd.backward([d1, d2], [cu(g1), cu(g2)])
    w1, w2 = orc.chamfer_grad(c1, c2, i1, i2, g1, g2)
    np.testing.assert_allclose(npy(x1.grad), w1, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(npy(x2.grad), w2, rtol=1e-4, atol=1e-4)


def test_chamfer_indices_bit_exact_with_duplicates():
    c1 = np.zeros((1, 4, 3), np.float32)
    c2 = np.tile(np.array([[1, 0, 0]], np.float32), (1, 1500, 1))   # every candidate ties
    lib = _lib.lib()
    x1, x2 = cu(c1), cu(c2)
    d1 = torch.empty(1, 4, device=DEV); d2 = torch.empty(1, 1500, device=DEV)
    i1 = torch.empty(1, 4, dtype=torch.int32, device=DEV); i2 = torch.empty(1, 1500, dtype=torch.int32, device=DEV)
    _lib.call("tpk_chamfer_dist_f32", 1, 4, _lib.ptr(x1), 1500, _lib.ptr(x2), _lib.ptr(d1), _lib.ptr(d2),
              _lib.ptr(i1), _lib.ptr(i2), _lib.stream_of(x1))
    o1, o2, oi1, oi2 = orc.chamfer(c1, c2)
    np.testing.assert_array_equal(npy(i1), oi1)
    np.testing.assert_array_equal(npy(i2), oi2)
    assert npy(i1).tolist() == [[0, 0, 0, 0]]


@pytest.mark.parametrize("case", ["sphere_pair", "sphere_pair_large", "one_side_small", "duplicates", "lattice_ties",
                                  "nonfinite", "planar"])
def test_chamfer_grid_path_matches_oracle_and_scan(case, monkeypatch):
    """Clouds of 1024+ points search the other cloud's uniform grid (in shared memory up to 8192
    points, in global scratch above): same distances (bits) and same indices as the all-pairs
    scan and the oracle, also where many candidates tie."""
    rng = np.random.default_rng(len(case))
    B = 2
    if case == "sphere_pair":
        c1, c2 = data.chamfer_pair(B, 6000, seed=4100)
        c1, c2 = c1.numpy().copy(), c2.numpy().copy()
    elif case == "sphere_pair_large":
        c1, c2 = data.chamfer_pair(B, 11000, seed=4103)
        c1, c2 = c1.numpy().copy(), c2[:, :9000].numpy().copy()
    elif case == "one_side_small":
        c1, c2 = data.chamfer_pair(B, 5000, seed=4101)
        c1, c2 = c1.numpy().copy(), c2[:, :700].numpy().copy()   # only one direction has a grid
    elif case == "duplicates":
        c2 = rng.uniform(-1, 1, (B, 4500, 3)).astype(np.float32)
        c2[:, 2000:3000] = c2[:, :1000]                          # every nearest neighbour twice
        c1 = (c2[:, ::2] + rng.normal(0, 1e-3, (B, 2250, 3))).astype(np.float32)
        c1 = np.concatenate([c1, c2[:, :2000]], axis=1)          # and queries that sit on candidates
    elif case == "lattice_ties":
        c1 = (rng.integers(0, 20, (B, 4096, 3)) / 8).astype(np.float32)
        c2 = (rng.integers(0, 10, (B, 5000, 3)) / 4).astype(np.float32)
    elif case == "nonfinite":
        c1, c2 = data.chamfer_pair(B, 4096, seed=4102)
        c1, c2 = c1.numpy().copy(), c2.numpy().copy()
        c1[0, 5, 1] = np.inf       # a query without a cell
        c2[1, 77, 0] = np.inf      # a cloud without a grid
    else:
        c1 = rng.uniform(0, 1, (B, 4200, 3)).astype(np.float32)
        c2 = rng.uniform(0, 1, (B, 4300, 3)).astype(np.float32)
        c1[..., 2] = 0.5
        c2[..., 2] = 0.5
    n, m = c1.shape[1], c2.shape[1]
    assert _lib.lib().tpk_chamfer_dist_scratch_bytes(B, n, m) > 0
    results = []
    # default (grid in shared memory, by layers above 8192 points), grid in global memory, scan
    for env in (None, "nn_global_grid", "chamfer_scan"):
        data.use_paths(monkeypatch, env)
        x1, x2 = cu(c1).requires_grad_(True), cu(c2).requires_grad_(True)
        d1, d2 = cd.ChamferFunction.apply(x1, x2)
        torch.autograd.backward([d1, d2], [torch.ones_like(d1), torch.ones_like(d2)])
        results.append((npy(d1), npy(d2), npy(x1.grad), npy(x2.grad)))
    if case != "nonfinite":  # the oracle and the kernels agree on finite data; non-finite: grid == scan
        o1, o2, _, _ = orc.chamfer(c1, c2)
        same_bits(results[0][0], o1)
        same_bits(results[0][1], o2)
    with np.errstate(invalid="ignore"):
        for other in results[1:]:
            same_bits(results[0][0], other[0])
            same_bits(results[0][1], other[1])
            # gradients are summed with atomics (order varies): equal up to rounding
            np.testing.assert_allclose(results[0][2], other[2], rtol=1e-4, atol=1e-4)
            np.testing.assert_allclose(results[0][3], other[3], rtol=1e-4, atol=1e-4)
    # the indices themselves, through the C ABI: grid + scratch against the plain scan
    data.use_paths(monkeypatch)
    x1, x2 = cu(c1), cu(c2)
    out = []
    for use_ws in (True, False):
        d1 = torch.empty(B, n, device=DEV); d2 = torch.empty(B, m, device=DEV)
        i1 = torch.empty(B, n, dtype=torch.int32, device=DEV); i2 = torch.empty(B, m, dtype=torch.int32, device=DEV)
        if use_ws:
            need = _lib.lib().tpk_chamfer_dist_scratch_bytes(B, n, m)
            scratch = torch.empty(need, dtype=torch.uint8, device=DEV)
            _lib.call("tpk_chamfer_dist_f32_ws", B, n, _lib.ptr(x1), m, _lib.ptr(x2), _lib.ptr(d1), _lib.ptr(d2),
                      _lib.ptr(i1), _lib.ptr(i2), _lib.ptr(scratch), need, _lib.stream_of(x1))
        else:
            _lib.call("tpk_chamfer_dist_f32", B, n, _lib.ptr(x1), m, _lib.ptr(x2), _lib.ptr(d1), _lib.ptr(d2),
                      _lib.ptr(i1), _lib.ptr(i2), _lib.stream_of(x1))
        out.append((npy(i1), npy(i2)))
    np.testing.assert_array_equal(out[0][0], out[1][0])
    np.testing.assert_array_equal(out[0][1], out[1][1])
    if case != "nonfinite":
        _, _, oi1, oi2 = orc.chamfer(c1, c2)
        np.testing.assert_array_equal(out[0][0], oi1)
        np.testing.assert_array_equal(out[0][1], oi2)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def test_chamfer_float64_gradcheck():
    g = data.gen(11)
    x = torch.rand(4, 64, 3, generator=g).double().to(DEV).requires_grad_(True)
    y = torch.rand(4, 128, 3, generator=g).double().to(DEV).requires_grad_(True)
    assert torch.autograd.gradcheck(cd.ChamferFunction.apply, [x, y])
    o1, o2, _, _ = orc.chamfer(x.detach().cpu(), y.detach().cpu())
    d1, d2 = cd.ChamferFunction.apply(x, y)
    np.testing.assert_allclose(npy(d1), o1, rtol=1e-12)
    np.testing.assert_allclose(npy(d2), o2, rtol=1e-12)


# ------------------------------------------------- the CPU-runnable plumbing configuration

def test_config1_plumbing_end_to_end():
    x, y, feat = data.cfg1_plumbing()
    xc, yc = cu(x), cu(y)
    idx, dist = tpk.ball_query(0.2, 32, xc, yc, mode="dense")
    oi, od = orc.ball_query_dense(0.2, 32, x, y)
    np.testing.assert_array_equal(npy(idx), oi)
    same_bits(npy(dist), od)
    ki, kd = tpk.knn(xc, yc, 3)
    oki, okd = orc.knn(x, y, 3)
    np.testing.assert_array_equal(npy(ki), oki)
    same_bits(npy(kd), okd)
    d, i3 = tpk.three_nn(xc, yc)
    od2, oi3 = orc.three_nn(x, y)
    np.testing.assert_array_equal(npy(i3), oi3)
    w = 1.0 / (d + 1e-8)
    w = w / w.sum(2, keepdim=True)
    out = tpk.three_interpolate(cu(feat), i3, w.contiguous())
    np.testing.assert_allclose(npy(out), orc.three_interpolate(feat, oi3, npy(w)), rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------ empty and degenerate inputs

def test_empty_and_degenerate_inputs():
    z3 = torch.zeros((0, 16, 3), device=DEV)
    assert tuple(tpk.furthest_point_sample(z3, 4).shape) == (0, 4)
    x = cu(data.unit_ball(2, 64, seed=1))
    # npoint == N: every valid point is selected exactly once before repeats start
    idx = npy(tpk.furthest_point_sample(x, 64))
    np.testing.assert_array_equal(idx, orc.fps(x.cpu(), 64))
    # no centres / no candidates / nsample 0
    i, d = tpk.ball_query(0.5, 8, x, torch.zeros((2, 0, 3), device=DEV))
    assert tuple(i.shape) == (2, 0, 8) and tuple(d.shape) == (2, 0, 8)
    i, d = tpk.ball_query(0.5, 8, torch.zeros((2, 0, 3), device=DEV), x[:, :5].contiguous())
    assert (npy(i) == 0).all() and (npy(d) == -1).all()
    i, d = tpk.ball_query(0.5, 4, torch.zeros((0, 3), device=DEV), x[0, :5].contiguous(), mode="partial_dense",
                          batch_x=torch.zeros((0,), dtype=torch.long, device=DEV),
                          batch_y=torch.zeros((5,), dtype=torch.long, device=DEV))
    assert (npy(i) == -1).all() and (npy(d) == -1).all()
    # three_nn with no known points: +inf distances, index 0
    dist, i3 = tpk.three_nn(x, torch.zeros((2, 0, 3), device=DEV))
    assert np.isinf(npy(dist)).all() and (npy(i3) == 0).all()
    # grouping / interpolation with empty outputs, gradient of an empty grouping is zero
    f = cu(torch.randn(2, 3, 64)).requires_grad_(True)
    g = tpk.grouping_operation(f, torch.zeros((2, 0, 4), dtype=torch.long, device=DEV))
    assert tuple(g.shape) == (2, 3, 0, 4)
    g.sum().backward()
    assert (npy(f.grad) == 0).all()
    # chamfer against an empty cloud: the reference leaves zeros
    d1, d2 = cd.ChamferFunction.apply(x, torch.zeros((2, 0, 3), device=DEV))
    assert (npy(d1) == 0).all() and tuple(d2.shape) == (2, 0)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


# ------------------------------------------------------------- indices that address nothing

@pytest.mark.parametrize("path", [None, "gather_direct"])
def test_grouping_skips_indices_out_of_range(path, monkeypatch):
    """An index outside [0, n) reads nothing (the output element is 0) and is recorded in the
    status word.  The bad values are chosen so that, without the guard, they would still land
    inside memory this test owns: n is the first element of the next feature row (rows of a
    CTA are adjacent in shared memory, and the tensor is a slice of a larger allocation), -1
    the last element of the row before."""
    data.use_paths(monkeypatch, path)
    B, C, n, npoint, ns = 2, 8, 4096, 512, 32
    g = data.gen(11)
    big = torch.randn(B * C * n + 2 * n, generator=g).to(DEV)
    feat = big[n:n + B * C * n].view(B, C, n)          # owned memory on both sides of the tensor
    idx = torch.randint(0, n, (B, npoint, ns), generator=g).to(DEV)
    good = npy(tpk.grouping_operation(feat, idx))
    bad = idx.clone()
    bad[0, 3, 5] = n
    bad[1, 100, 0] = -1
    bad[1, 7, 31] = 1 << 40
    out, status = _guarded(lambda: tpk.grouping_operation(feat, bad))
    assert status == 2
    out = npy(out)
    mask = np.zeros((B, npoint, ns), bool)
    mask[0, 3, 5] = mask[1, 100, 0] = mask[1, 7, 31] = True
    assert (out[:, :, :, :][np.broadcast_to(mask[:, None], out.shape)] == 0).all()
    keep = ~np.broadcast_to(mask[:, None], out.shape)
    np.testing.assert_array_equal(out[keep], good[keep])


def test_grouping_grad_sorted_drops_indices_out_of_range():
    """Same contract through the inverted index: a bad index adds nothing, sets the status bit,
    and nothing outside the result tensor is written."""
    B, C, n, npoint, ns = 2, 8, 10000, 256, 32
    g = data.gen(13)
    idx = torch.randint(0, n, (B, npoint, ns), generator=g)
    gout = torch.randn(B, C, npoint, ns, generator=g)
    bad = idx.clone()
    bad[0, 3, 5] = n
    bad[1, 100, 0] = -1
    bad[1, 255, 31] = 1 << 40
    big = torch.zeros(B * C * n + 2 * n, device=DEV)
    grad = big[n:n + B * C * n].view(B, C, n)
    gout_d, bad_d = cu(gout), cu(bad)
    need = _lib.lib().tpk_grouping_grad_scratch_bytes(B, C, n, npoint, ns)
    assert need > 0
    scratch = torch.empty(need, dtype=torch.uint8, device=DEV)

    def run():
        _lib.call("tpk_grouping_grad_ws", B, C, n, npoint, ns, _lib.ptr(gout_d), _lib.ptr(bad_d), _lib.ptr(grad),
                  _lib.ptr(scratch), need, _lib.stream_of(grad))
        return grad
    _, status = _guarded(run)
    assert status == 2
    w = gout.clone().numpy()
    w[0, :, 3, 5] = 0
    w[1, :, 100, 0] = 0
    w[1, :, 255, 31] = 0
    np.testing.assert_allclose(npy(grad), orc.grouping_grad(w, idx.numpy(), n), rtol=1e-4, atol=1e-4)
    assert float(big[:n].abs().max()) == 0 and float(big[n + B * C * n:].abs().max()) == 0


@pytest.mark.parametrize("path", [None, "scatter_global"])
def test_grouping_grad_drops_indices_out_of_range(path, monkeypatch):
    data.use_paths(monkeypatch, path)
    B, C, n, npoint, ns = 2, 8, 2048, 256, 32
    g = data.gen(12)
    idx = torch.randint(0, n, (B, npoint, ns), generator=g)
    gout = torch.randn(B, C, npoint, ns, generator=g)
    bad = idx.clone()
    bad[0, 3, 5] = n       # the next row of the CTA's shared-memory accumulator
    bad[1, 100, 0] = -1
    big = torch.zeros(B * C * n + 2 * n, device=DEV)
    grad = big[n:n + B * C * n].view(B, C, n)
    gout_d, bad_d = cu(gout), cu(bad)  # kept alive: the call only sees their addresses

    def run():
        _lib.call("tpk_grouping_grad", B, C, n, npoint, ns, _lib.ptr(gout_d), _lib.ptr(bad_d), _lib.ptr(grad),
                  _lib.stream_of(grad))
        return grad
    _, status = _guarded(run)
    assert status == 2
    # everything but the two dropped contributions, and nothing outside the tensor
    want_idx = idx.clone().numpy()
    w = gout.clone().numpy()
    w[0, :, 3, 5] = 0
    w[1, :, 100, 0] = 0
    np.testing.assert_allclose(npy(grad), orc.grouping_grad(w, want_idx, n), rtol=1e-4, atol=1e-4)
    assert float(big[:n].abs().max()) == 0 and float(big[n + B * C * n:].abs().max()) == 0


@pytest.mark.parametrize("path", [None, "gather_direct", "scatter_global"])
def test_three_interpolate_skips_indices_out_of_range(path, monkeypatch):
    data.use_paths(monkeypatch, path)
    B, C, m, n = 2, 16, 512, 2048
    g = data.gen(13)
    big = torch.randn(B * C * m + 2 * m, generator=g).to(DEV)
    feat = big[m:m + B * C * m].view(B, C, m).requires_grad_(True)
    idx = torch.randint(0, m, (B, n, 3), generator=g).int()
    w = torch.rand(B, n, 3, generator=g)
    bad = idx.clone()
    bad[0, 9, 1] = m
    bad[1, 1000, 2] = -1
    out, status = _guarded(lambda: tpk.three_interpolate(feat, cu(bad), cu(w)))
    assert status == 2
    w0 = w.clone()
    w0[0, 9, 1] = 0
    w0[1, 1000, 2] = 0
    np.testing.assert_allclose(npy(out), orc.three_interpolate(npy(feat), idx.numpy(), w0.numpy()), rtol=1e-5, atol=1e-6)
    gout = torch.randn(B, C, n, generator=g)
    _, status = _guarded(lambda: out.backward(cu(gout)))
    assert status == 2
    np.testing.assert_allclose(npy(feat.grad), orc.three_interpolate_grad(gout, idx.numpy(), w0.numpy(), m),
                               rtol=1e-4, atol=1e-4)


def test_debug_mode_raises_on_bad_inputs(monkeypatch):
    """TPK_B200_DEBUG: segment vectors are validated on the host (as the reference's CPU path
    does) and a skipped index becomes an exception right after the call."""
    monkeypatch.setenv("TPK_B200_DEBUG", "1")
    x = cu(data.unit_ball(1, 100, seed=1)[0])
    with pytest.raises(RuntimeError, match="same number of samples"):
        tpk.ball_query(1.0, 2, x, x[:1].contiguous(), mode="PARTIAL_DENSE",
                       batch_x=cu(torch.tensor([0] * 50 + [1] * 50)), batch_y=cu(torch.tensor([0])))
    with pytest.raises(RuntimeError, match="sorted"):
        tpk.knn(x, x[:2].contiguous(), 2, batch_support=cu(torch.tensor([1] * 50 + [0] * 50)),
                batch_pos=cu(torch.tensor([0, 1])))
    feat = cu(torch.randn(1, 4, 100))
    idx = cu(torch.full((1, 8, 4), 100, dtype=torch.long))
    with pytest.raises(RuntimeError, match="index outside"):
        tpk.grouping_operation(feat, idx)
    assert _lib.device_status() == 0


def test_backward_accepts_views_at_odd_offsets():
    """grad_out / idx that are contiguous views starting off a 16-byte boundary work in the
    backward passes as they do in the forward ones."""
    g = data.gen(14)
    B, C, n, npoint, ns = 1, 4, 300, 37, 3
    idx = torch.randint(0, n, (B * npoint * ns + 1,), generator=g).to(DEV)[1:].view(B, npoint, ns)
    gout = torch.randn(B * C * npoint * ns + 1, generator=g).to(DEV)[1:].view(B, C, npoint, ns)
    grad = torch.empty(B, C, n, device=DEV)
    _lib.call("tpk_grouping_grad", B, C, n, npoint, ns, _lib.ptr(gout), _lib.ptr(idx), _lib.ptr(grad), _lib.stream_of(grad))
    np.testing.assert_allclose(npy(grad), orc.grouping_grad(npy(gout), npy(idx), n), rtol=1e-4, atol=1e-4)
    m, nn = 64, 101
    idx3 = torch.randint(0, m, (B * nn * 3 + 1,), generator=g).int().to(DEV)[1:].view(B, nn, 3)
    w = torch.rand(B * nn * 3 + 1, generator=g).to(DEV)[1:].view(B, nn, 3)
    go = torch.randn(B * C * nn + 1, generator=g).to(DEV)[1:].view(B, C, nn)
    gp = torch.empty(B, C, m, device=DEV)
    _lib.call("tpk_three_interpolate_grad", B, C, nn, m, _lib.ptr(go), _lib.ptr(idx3), _lib.ptr(w), _lib.ptr(gp),
              _lib.stream_of(gp))
    np.testing.assert_allclose(npy(gp), orc.three_interpolate_grad(npy(go), npy(idx3), npy(w), m), rtol=1e-4, atol=1e-4)
