"""Generates tests/golden/*.npz by running the REFERENCE implementation on seeded inputs.

Run from the repository root, in a container that has the reference tree:

    make -C oracle ref_cpu            # reference cpu/src/*.cpp -> oracle/_ref/points_cpu.so
    python tests/golden/make_golden.py [/path/to/reference]

The reference's Python layer (torch_points_kernels/*.py) is imported from the reference
tree and its compiled CPU extension from oracle/_ref; nothing of either is copied.
The fixtures hold inputs and the reference's outputs; tests compare the CPU oracle and
the CUDA kernels against them.  Only functions whose CPU semantics equal the CUDA
semantics on the given inputs are recorded as exact; ball-query results are recorded
sorted by distance (sort=True) and compared as sets, as the reference's own tests do.
"""
import os
import sys
import types

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
OUT = os.path.join(ROOT, "tests", "golden")


def import_reference():
    # a package whose modules come from the reference tree and whose extension comes from oracle/_ref
    pkg = types.ModuleType("torch_points_kernels")
    pkg.__path__ = [os.path.join(REF, "torch_points_kernels"), os.path.join(ROOT, "oracle", "_ref")]
    sys.modules["torch_points_kernels"] = pkg
    import torch_points_kernels.torchpoints as tp  # noqa: E402
    import torch_points_kernels.points_cpu as tpcpu  # noqa: E402

    return tp, tpcpu


def main():
    tp, tpcpu = import_reference()
    g = torch.Generator().manual_seed(20240607)

    # ---- plumbing case: the shape family of the CPU-runnable configuration, scaled down
    B, N, M, C = 2, 768, 192, 8
    x = torch.rand(B, N, 3, generator=g)
    y = torch.stack([x[b][torch.randperm(N, generator=g)[:M]] for b in range(B)]).contiguous()
    feat = torch.randn(B, C, M, generator=g)

    knn3_idx, knn3_d2 = tp.knn(x, y, 3)
    knn16_idx, knn16_d2 = tp.knn(x, y, 16)
    nn_dist, nn_idx = tp.three_nn(x, y)  # unknown = x, known = y (CPU path: kNN k=3)
    w = 1.0 / (nn_dist + 1e-8)
    w = w / w.sum(2, keepdim=True)
    f = feat.clone().requires_grad_(True)
    interp = tp.three_interpolate(f, nn_idx, w)
    gout = torch.randn(interp.shape, generator=g)
    interp.backward(gout)
    interp_grad = f.grad.clone()

    bq_idx, bq_d2 = tp.ball_query(0.2, 64, x, y, mode="dense", sort=True)

    gfeat = torch.randn(B, C, N, generator=g).requires_grad_(True)
    gidx = torch.randint(0, N, (B, 48, 16), generator=g)
    grouped = tp.grouping_operation(gfeat, gidx)
    ggout = torch.randn(grouped.shape, generator=g)
    grouped.backward(ggout)

    fps_idx = tpcpu.fps(x, 64, False)

    np.savez_compressed(
        os.path.join(OUT, "plumbing.npz"),
        x=x.numpy(), y=y.numpy(), feat=feat.numpy(),
        knn3_idx=knn3_idx.numpy(), knn3_d2=knn3_d2.numpy(),
        knn16_idx=knn16_idx.numpy(), knn16_d2=knn16_d2.numpy(),
        nn_dist=nn_dist.numpy(), nn_idx=nn_idx.numpy(), weight=w.numpy(),
        interp=interp.detach().numpy(), interp_gout=gout.numpy(), interp_grad=interp_grad.numpy(),
        bq_radius=np.float32(0.2), bq_nsample=np.int64(64),
        bq_idx=bq_idx.numpy(), bq_d2=bq_d2.numpy(),
        gfeat=gfeat.detach().numpy(), gidx=gidx.numpy(), grouped=grouped.detach().numpy(),
        grouped_gout=ggout.numpy(), grouped_grad=gfeat.grad.numpy(),
        fps_idx=fps_idx.numpy(),
    )

    # ---- packed segments: 3 segments of different size, every segment has queries
    sizes = [300, 150, 450]
    px = torch.cat([torch.rand(s, 3, generator=g) + 2.0 * i for i, s in enumerate(sizes)])
    bx = torch.cat([torch.full((s,), i, dtype=torch.long) for i, s in enumerate(sizes)])
    qsel = torch.cat([torch.randperm(s, generator=g)[: s // 5].sort().values + sum(sizes[:i])
                      for i, s in enumerate(sizes)])
    py = px[qsel].contiguous()
    by = bx[qsel].contiguous()
    pidx, pd2 = tp.ball_query(0.15, 32, px, py, mode="partial_dense", batch_x=bx, batch_y=by, sort=True)
    np.savez_compressed(
        os.path.join(OUT, "partial.npz"),
        x=px.numpy(), y=py.numpy(), batch_x=bx.numpy(), batch_y=by.numpy(),
        radius=np.float32(0.15), nsample=np.int64(32), idx=pidx.numpy(), d2=pd2.numpy(),
    )
    print("wrote", os.listdir(OUT))


if __name__ == "__main__":
    main()
