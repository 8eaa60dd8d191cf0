"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations.  Everything is generated on the CPU with a torch.Generator so
that the oracle and the GPU see identical bits; sizes are parameters so that tests can
run scaled-down versions of the same distributions."""
import math

import torch


def gen(seed):
    return torch.Generator().manual_seed(int(seed))


def cfg1_plumbing(B=4, N=4096, M=1024, C=64, seed=1000):
    g = gen(seed)
    x = torch.rand(B, N, 3, generator=g)
    y = torch.stack([x[b][torch.randperm(N, generator=g)[:M]] for b in range(B)]).contiguous()
    feat = torch.randn(B, C, M, generator=g)
    return x, y, feat


def unit_ball(B, N, seed=2000):
    """Uniform in the unit ball: direction = normalised randn, radius = rand^(1/3)."""
    g = gen(seed)
    d = torch.randn(B, N, 3, generator=g)
    d = d / d.norm(dim=2, keepdim=True)
    r = torch.rand(B, N, 1, generator=g) ** (1.0 / 3.0)
    return (d * r).contiguous()


def packed_planes(n_scenes=64, lo=20000, hi=200000, seed=3000, query_frac=0.1):
    """Scenes of points on 3-8 random axis-aligned 5 m x 5 m planes with 1 cm noise."""
    g = gen(seed)
    xs, bx, ys, by = [], [], [], []
    for s in range(n_scenes):
        n = int(torch.randint(lo, hi + 1, (1,), generator=g))
        planes = int(torch.randint(3, 9, (1,), generator=g))
        axis = torch.randint(0, 3, (planes,), generator=g)
        offset = torch.rand(planes, generator=g) * 5.0
        which = torch.randint(0, planes, (n,), generator=g)
        p = torch.rand(n, 3, generator=g) * 5.0
        p[torch.arange(n), axis[which]] = offset[which]
        p = p + torch.randn(n, 3, generator=g) * 0.01
        q = torch.randperm(n, generator=g)[: max(1, int(n * query_frac))].sort().values
        xs.append(p)
        bx.append(torch.full((n,), s, dtype=torch.long))
        ys.append(p[q])
        by.append(torch.full((q.numel(),), s, dtype=torch.long))
    return (torch.cat(xs).contiguous(), torch.cat(ys).contiguous(), torch.cat(bx), torch.cat(by))


def chamfer_pair(B=32, N=16384, seed=4000):
    g = gen(seed)
    c1 = torch.randn(B, N, 3, generator=g)
    c1 = c1 / c1.norm(dim=2, keepdim=True)
    c2 = c1.clone()
    k = int(0.3 * N)
    for b in range(B):
        rows = torch.randperm(N, generator=g)[:k]
        fresh = torch.randn(k, 3, generator=g)
        c2[b, rows] = fresh / fresh.norm(dim=1, keepdim=True)
    c2 = c2 + torch.randn(B, N, 3, generator=g) * 0.01
    for b in range(B):
        c2[b] = c2[b][torch.randperm(N, generator=g)]
    return c1.contiguous(), c2.contiguous()


def gaussian_mixture(B=8, N=1 << 20, seed=5000, comps=32):
    g = gen(seed)
    out = torch.empty(B, N, 3)
    for b in range(B):
        means = torch.rand(comps, 3, generator=g)
        sig = torch.exp(torch.rand(comps, 3, generator=g) * (math.log(0.2) - math.log(0.01)) + math.log(0.01))
        which = torch.randint(0, comps, (N,), generator=g)
        out[b] = means[which] + torch.randn(N, 3, generator=g) * sig[which]
    return out.contiguous()
