"""Cross-path consistency on random shapes: every search op through its default kernels (grids,
sorted copies, several samples per exchange) against the scan kernels of the same library, which
the parity tests pin to the oracle at fixed shapes; gathers and scatters against torch.  Shapes are
log-uniform with a bias to powers of two and their neighbours, where kernel plans change."""
import math
import os
import random

import pytest
import torch

import torch_points_kernels_b200 as tpk
from torch_points_kernels_b200 import _lib
from torch_points_kernels_b200.chamfer_dist import ChamferFunction

pytestmark = pytest.mark.gpu
dev = "cuda"


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes_agree_across_kernel_families(seed, monkeypatch):
    rnd = random.Random(seed)
    failures = []

    def hook(tokens):
        if tokens:
            monkeypatch.setenv("TPK_B200_TEST", tokens)
        else:
            monkeypatch.delenv("TPK_B200_TEST", raising=False)

    def pick(choices):
        return rnd.choice(choices)

    def size(lo, hi):
        v = int(round(math.exp(rnd.uniform(math.log(lo), math.log(hi)))))
        if rnd.random() < 0.3:
            p = 1 << max(0, v.bit_length() - 1)
            v = p + pick([-1, 0, 1, 0])
        return max(lo, min(hi, v))

    def cloud(B, N, g):
        kind = pick(["ball", "cube", "clumps"])
        if kind == "ball":
            d = torch.randn(B, N, 3, generator=g)
            d = d / d.norm(dim=2, keepdim=True)
            return (d * torch.rand(B, N, 1, generator=g) ** (1 / 3)).contiguous()
        if kind == "cube":
            return torch.rand(B, N, 3, generator=g) * 2 - 1
        c = torch.rand(B, 8, 3, generator=g) * 2 - 1
        return (c[:, torch.randint(0, 8, (N,), generator=g)] + 0.05 * torch.randn(B, N, 3, generator=g)).contiguous()

    def check(name, shape, fn):
        try:
            ok = fn()
            torch.cuda.synchronize()
            status = _lib.device_status()
            if not ok or status != 0:
                failures.append((name, shape, "mismatch" if not ok else "status %d" % status))
        finally:
            hook(None)

    iters = 120
    for it in range(iters):
        g = torch.Generator().manual_seed(seed * 100003 + it)
        op = pick(["fps", "ball", "three_nn", "knn", "group", "interp", "chamfer", "sa_group", "ball_partial", "fps_big"])
        if op == "fps":
            B, N = size(1, 20), size(1, 40000)
            m = size(1, min(N, 3000))
            x = cloud(B, N, g).to(dev)
            def f():
                hook(None); a = tpk.furthest_point_sample(x, m)
                hook("fps_unsorted"); b = tpk.furthest_point_sample(x, m)
                hook("fps_sorted,fps_single"); c = tpk.furthest_point_sample(x, m)
                return bool(torch.equal(a, b) and torch.equal(a, c))
            check(op, (B, N, m), f)
        elif op == "fps_big":
            # clouds beyond the on-chip kernels: chunk-skipping kernel on the sorted copy against the
            # kernel that keeps every running minimum in global memory
            B, N = size(1, 3), size(131073, 400000)
            m = size(1, 200)
            x = cloud(B, N, g).to(dev)
            def f():
                hook(None); a = tpk.furthest_point_sample(x, m)
                hook("fps_unsorted"); b = tpk.furthest_point_sample(x, m)
                return bool(torch.equal(a, b))
            check(op, (B, N, m), f)
        elif op == "ball":
            B, N, M = size(1, 8), size(1, 30000), size(1, 3000)
            ns = pick([1, 3, 16, 32, 64]); r = pick([0.05, 0.1, 0.3, 1.0])
            x = cloud(B, N, g).to(dev); c = cloud(B, M, g).to(dev)
            def f():
                hook(None); a, ad = tpk.ball_query(r, ns, x, c, mode="dense")
                hook("ball_query_scan"); b, bd = tpk.ball_query(r, ns, x, c, mode="dense")
                return bool(torch.equal(a, b) and torch.equal(ad, bd))
            check(op, (B, N, M, ns, r), f)
        elif op == "three_nn":
            B, n, m = size(1, 8), size(3, 20000), size(3, 9000)
            u = cloud(B, n, g).to(dev); k = cloud(B, m, g).to(dev)
            def f():
                hook(None); d, i = tpk.three_nn(u, k)
                hook("three_nn_scan"); d2, i2 = tpk.three_nn(u, k)
                return bool(torch.equal(d, d2) and torch.equal(i, i2))
            check(op, (B, n, m), f)
        elif op == "knn":
            B, ns_, nq = size(1, 6), size(1, 20000), size(1, 3000)
            k = min(ns_, pick([1, 3, 8, 16, 32]))
            s = cloud(B, ns_, g).to(dev); q = cloud(B, nq, g).to(dev)
            def f():
                hook(None); i, d = tpk.knn(s, q, k)
                hook("knn_scan"); i2, d2 = tpk.knn(s, q, k)
                return bool(torch.equal(d, d2) and torch.equal(i, i2))
            check(op, (B, ns_, nq, k), f)
        elif op == "group":
            B, C, N, P, S = size(1, 8), size(1, 200), size(1, 40000), size(1, 5000), pick([1, 3, 8, 16, 32, 64])
            feat = torch.randn(B, C, N, generator=g).to(dev)
            idx = torch.randint(0, N, (B, P, S), generator=g).to(dev)
            gout = torch.randn(B, C, P, S, generator=g).to(dev)
            def f():
                out = tpk.grouping_operation(feat, idx)
                ref = torch.gather(feat, 2, idx.view(B, 1, P * S).expand(B, C, P * S)).view(B, C, P, S)
                gb = tpk.torchpoints.grouping_backward(gout, idx, N)
                want = torch.zeros(B, C, N, device=dev, dtype=torch.float64).scatter_add_(2, idx.view(B, 1, P * S).expand(B, C, P * S), gout.double().view(B, C, P * S))
                tol = 1e-4 * max(1.0, float(want.abs().max()))
                return bool(torch.equal(out, ref) and (gb.double() - want).abs().max() <= tol)
            check(op, (B, C, N, P, S), f)
        elif op == "interp":
            B, C, m, n = size(1, 8), size(1, 200), size(1, 20000), size(1, 30000)
            p = torch.randn(B, C, m, generator=g).to(dev)
            i3 = torch.randint(0, m, (B, n, 3), generator=g).int().to(dev)
            w = torch.rand(B, n, 3, generator=g).to(dev)
            gout = torch.randn(B, C, n, generator=g).to(dev)
            def f():
                up = tpk.three_interpolate(p, i3, w)
                gath = torch.gather(p, 2, i3.long().view(B, 1, n * 3).expand(B, C, n * 3)).view(B, C, n, 3)
                want = (gath.double() * w.double().unsqueeze(1)).sum(-1)
                gb = tpk.torchpoints.three_interpolate_backward(gout, i3, w, m)
                wantg = torch.zeros(B, C, m, device=dev, dtype=torch.float64).scatter_add_(
                    2, i3.long().view(B, 1, n * 3).expand(B, C, n * 3), (gout.double().unsqueeze(-1) * w.double().unsqueeze(1)).reshape(B, C, n * 3))
                tol = 1e-4 * max(1.0, float(wantg.abs().max()))
                return bool((up.double() - want).abs().max() <= 1e-4 * max(1.0, float(want.abs().max())) and (gb.double() - wantg).abs().max() <= tol)
            check(op, (B, C, m, n), f)
        elif op == "chamfer":
            B, n, m = size(1, 8), size(1, 12000), size(1, 12000)
            a = cloud(B, n, g).to(dev); b = cloud(B, m, g).to(dev)
            def f():
                hook(None); d1, d2 = ChamferFunction.apply(a, b)
                hook("chamfer_scan"); e1, e2 = ChamferFunction.apply(a, b)
                return bool(torch.equal(d1, e1) and torch.equal(d2, e2))
            check(op, (B, n, m), f)
        elif op == "sa_group":
            B, N, M, C = size(1, 6), size(8, 20000), size(1, 2000), size(1, 80)
            M = min(M, N); ns = pick([8, 16, 32]); r = pick([0.1, 0.3])
            x = cloud(B, N, g).to(dev); feat = torch.randn(B, C, N, generator=g).to(dev)
            def f():
                fi = tpk.furthest_point_sample(x, M)
                nx, idx, out = tpk.sa_group(x, feat, fi, r, ns)
                c_xyz = torch.gather(x, 1, fi.long().unsqueeze(-1).expand(-1, -1, 3)).contiguous()
                nb, _ = tpk.ball_query(r, ns, x, c_xyz, mode="dense")
                rel = tpk.grouping_operation(x.transpose(1, 2).contiguous(), nb) - c_xyz.transpose(1, 2).unsqueeze(-1)
                want = torch.cat([rel, tpk.grouping_operation(feat, nb)], dim=1)
                return bool(torch.equal(idx, nb) and torch.equal(out, want) and torch.equal(nx, c_xyz))
            check(op, (B, N, M, C, ns, r), f)
        elif op == "ball_partial":
            nseg = size(1, 12)
            sizes_x = [size(1, 6000) for _ in range(nseg)]; sizes_y = [size(1, 600) for _ in range(nseg)]
            x = torch.cat([cloud(1, s, g)[0] for s in sizes_x]).to(dev); y = torch.cat([cloud(1, s, g)[0] for s in sizes_y]).to(dev)
            bx = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(sizes_x)]).to(dev)
            by = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(sizes_y)]).to(dev)
            ns = pick([4, 16, 64]); r = pick([0.05, 0.2])
            def f():
                hook(None); a, ad = tpk.ball_query(r, ns, x, y, mode="partial_dense", batch_x=bx, batch_y=by)
                hook("ball_query_scan"); b, bd = tpk.ball_query(r, ns, x, y, mode="partial_dense", batch_x=bx, batch_y=by)
                return bool(torch.equal(a, b) and torch.equal(ad, bd))
            check(op, (sizes_x, sizes_y, ns, r), f)
    assert not failures, failures
