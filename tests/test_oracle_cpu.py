"""CPU tests: the oracle against the reference's known-answer vectors and against
fixtures produced by the reference itself (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from oracle import oracle as orc


def _f(a):
    return np.asarray(a, dtype=np.float32)


def test_known_ball_query_dense(known_answers):
    ka = known_answers["ball_query_dense_cuda"]
    idx, dist = orc.ball_query_dense(ka["radius"], ka["nsample"], _f(ka["x"]), _f(ka["y"]))
    assert idx.tolist() == ka["idx"]
    np.testing.assert_allclose(dist, _f(ka["dist"]), rtol=0, atol=1e-6)


def test_known_ball_query_dense_sets(known_answers):
    # the CPU known answer is distance-sorted; the index-order rule must find the same sets
    ka = known_answers["ball_query_dense_cpu_sorted"]
    x = _f(ka["x"])
    idx, _ = orc.ball_query_dense(ka["radius"], ka["nsample"], x, x)
    for got, want in zip(idx[0], ka["idx_sorted_by_distance"][0]):
        assert set(got.tolist()) == set(want)


@pytest.mark.parametrize("name", ["ball_query_partial_cuda", "ball_query_partial_cpu"])
def test_known_ball_query_partial(known_answers, name):
    ka = known_answers[name]
    idx, dist = orc.ball_query_partial(ka["radius"], ka["nsample"], _f(ka["x"]), _f(ka["y"]),
                                       ka["batch_x"], ka["batch_y"])
    assert idx.tolist() == ka["idx"]
    np.testing.assert_allclose(dist, _f(ka["dist"]), rtol=0, atol=1e-6)


def test_known_fps(known_answers):
    ka = known_answers["fps_start0"]
    assert orc.fps(_f(ka["points"]), ka["npoint"]).tolist() == ka["idx"]


def test_known_grouping(known_answers):
    ka = known_answers["grouping"]
    out = orc.grouping(_f(ka["features"]), np.asarray(ka["idx"], np.int64))
    np.testing.assert_array_equal(out, _f(ka["expected"]))


def test_known_knn(known_answers):
    ka = known_answers["knn"]
    idx, d2 = orc.knn(_f(ka["support"]), _f(ka["query"]), 3)
    assert idx.tolist() == ka["k3_idx"]
    np.testing.assert_array_equal(d2, _f(ka["k3_dist"]))
    idx, _ = orc.knn(_f(ka["support"]), _f(ka["query"]), 2)
    assert idx.tolist() == ka["k2_idx"]
    with pytest.raises(RuntimeError):
        orc.knn(_f(ka["support"]), _f(ka["query"]), ka["k_too_large"])


def test_known_chamfer(known_answers):
    ka = known_answers["chamfer"]
    d1, d2, _, _ = orc.chamfer(_f(ka["xyz1"]), _f(ka["xyz2"]))
    assert abs(float(d1.mean() + d2.mean()) - ka["dist"]) < 10 ** -ka["places"]
    x1 = _f(ka["xyz1"])[:, 1:]  # ignore_zeros drops the all-zero point of cloud 1
    d1, d2, _, _ = orc.chamfer(x1, _f(ka["xyz2"]))
    assert abs(float(d1.mean() + d2.mean()) - ka["dist_ignore_zeros"]) < 10 ** -ka["places"]


@pytest.fixture(scope="module")
def plumbing(golden_dir):
    return np.load(os.path.join(golden_dir, "plumbing.npz"))


def test_golden_knn_bit_exact(plumbing):
    for k in (3, 16):
        idx, d2 = orc.knn(plumbing["x"], plumbing["y"], k)
        np.testing.assert_array_equal(idx, plumbing["knn%d_idx" % k])
        np.testing.assert_array_equal(d2.view(np.int32), plumbing["knn%d_d2" % k].view(np.int32))


def test_golden_three_nn(plumbing):
    # reference CPU three_nn = kNN(k=3) with unfused arithmetic: same neighbours, distances to 1e-5
    d2, idx = orc.three_nn(plumbing["x"], plumbing["y"])
    np.testing.assert_array_equal(idx.astype(np.int64), plumbing["nn_idx"])
    np.testing.assert_allclose(np.sqrt(d2), plumbing["nn_dist"], rtol=1e-5, atol=1e-7)


def test_golden_interpolate(plumbing):
    out = orc.three_interpolate(plumbing["feat"], plumbing["nn_idx"], plumbing["weight"])
    np.testing.assert_allclose(out, plumbing["interp"], rtol=1e-5, atol=1e-6)
    grad = orc.three_interpolate_grad(plumbing["interp_gout"], plumbing["nn_idx"], plumbing["weight"],
                                      plumbing["feat"].shape[2])
    np.testing.assert_allclose(grad, plumbing["interp_grad"], rtol=1e-4, atol=1e-4)


def test_golden_grouping(plumbing):
    out = orc.grouping(plumbing["gfeat"], plumbing["gidx"])
    np.testing.assert_array_equal(out, plumbing["grouped"])
    grad = orc.grouping_grad(plumbing["grouped_gout"], plumbing["gidx"], plumbing["gfeat"].shape[2])
    np.testing.assert_allclose(grad, plumbing["grouped_grad"], rtol=1e-4, atol=1e-4)


def _sets_match(idx, d2, ref_idx, ref_d2, r2, strict):
    """Set equality per query, leaving out neighbours exactly on the radius (the
    reference CPU path is strict, the CUDA partial_dense rule is inclusive)."""
    for q in range(idx.shape[0]):
        got = {int(i) for i, d in zip(idx[q], d2[q]) if d >= 0 and (strict or d != r2)}
        want = {int(i) for i, d in zip(ref_idx[q], ref_d2[q]) if d >= 0}
        if got != want:
            return False
    return True


def test_golden_ball_query_dense_sets(plumbing):
    r, ns = float(plumbing["bq_radius"]), int(plumbing["bq_nsample"])
    ref_idx, ref_d2 = plumbing["bq_idx"], plumbing["bq_d2"]
    assert (ref_d2 >= 0).sum(-1).max() < ns  # no query is truncated, so sets are comparable
    idx, d2 = orc.ball_query_dense(r, ns, plumbing["x"], plumbing["y"])
    r2 = np.float32(r) * np.float32(r)
    for b in range(idx.shape[0]):
        assert _sets_match(idx[b], d2[b], ref_idx[b], ref_d2[b], r2, True)
    # index order and padding rule of the CUDA path
    cnt = (d2 >= 0).sum(-1)
    for b in range(idx.shape[0]):
        for q in range(idx.shape[1]):
            c = cnt[b, q]
            assert (np.diff(idx[b, q, :c]) > 0).all()
            assert (idx[b, q, c:] == (idx[b, q, 0] if c else 0)).all()


def test_golden_ball_query_partial_sets(golden_dir):
    p = np.load(os.path.join(golden_dir, "partial.npz"))
    r, ns = float(p["radius"]), int(p["nsample"])
    assert (p["d2"] >= 0).sum(-1).max() < ns
    idx, d2 = orc.ball_query_partial(r, ns, p["x"], p["y"], p["batch_x"], p["batch_y"])
    r2 = np.float32(r) * np.float32(r)
    assert _sets_match(idx, d2, p["idx"], p["d2"], r2, False)
    assert ((idx == -1) == (d2 == -1)).all()


def test_golden_fps(plumbing):
    # the reference CPU FPS (start 0) agrees with the CUDA rule when no point lies within
    # sqrt(1e-3) of the origin and no two distances tie
    x = plumbing["x"]
    assert ((x ** 2).sum(-1) > 2e-3).all()
    np.testing.assert_array_equal(orc.fps(x, plumbing["fps_idx"].shape[1]).astype(np.int64), plumbing["fps_idx"])


def test_fps_tie_rule_matches_rank_formula():
    """Replayed tree reduction == closed form: among equal maxima the winner minimises
    (bit-reversed (k mod bs), k div bs)."""
    rng = np.random.default_rng(7)
    for n in (3, 8, 37, 64, 300, 700, 1500):
        bs = orc.opt_n_threads(n)
        assert bs == min(512, 1 << (n.bit_length() - 1))
        L = bs.bit_length() - 1
        # all candidate points at the same distance from point 0: a regular simplex is not
        # needed, duplicates of one far point tie exactly
        pts = np.zeros((1, n, 3), np.float32)
        pts[0, 0] = (1.0, 1.0, 1.0)
        far = rng.choice(np.arange(1, n), size=max(1, (n - 1) // 2), replace=False)
        pts[0, 1:] = (1.0, 1.0, 1.5)
        pts[0, far] = (5.0, 1.0, 1.0)
        got = int(orc.fps(pts, 2)[0, 1])

        def rank(k):
            rev = int(format(k % bs, "0%db" % L)[::-1], 2) if L else 0
            return (rev, k // bs)

        assert got == min(far.tolist(), key=rank)


def test_fps_skips_points_near_origin():
    pts = np.array([[[1, 0, 0], [0.01, 0.01, 0.01], [-3, 0, 0], [0.5, 0, 0]]], np.float32)
    # point 1 has |p|^2 = 3e-4 <= 1e-3 and is never selected while others remain
    assert orc.fps(pts, 3)[0].tolist() == [0, 2, 3]
    # all points skipped: every round returns 0
    tiny = np.full((1, 5, 3), 0.001, np.float32)
    assert orc.fps(tiny, 4)[0].tolist() == [0, 0, 0, 0]
