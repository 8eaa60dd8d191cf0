"""Benchmark of the spatial-search hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Default workload "sa_fp_pipeline": the PointNet++ SSG set-abstraction / feature-propagation
stack on B=16 clouds of N=16384 points per GPU (FPS to 4096/1024/256/64, ball query radii
0.1/0.2/0.4/0.8 with nsample 32, grouping of C=64/128/256/512 features, three_nn +
three_interpolate back up every level, forward and backward), seeded synthetic data.
One step = one pass of that stack over one batch.  Prints ONE JSON line (rank 0).

--impl reference times the reference's own CPU implementation (its nanoflann / ATen
extension compiled from the reference sources into oracle/_ref, or the oracle port when
that is absent) on the host cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LEVELS = dict(npoint=[4096, 1024, 256, 64], radius=[0.1, 0.2, 0.4, 0.8], nsample=32, channels=[64, 128, 256, 512])
B_CLOUDS, N_POINTS = 16, 16384
METRIC = "sa_fp_pipeline_clouds_per_s"


# --------------------------------------------------------------------------- inputs

def make_inputs(B, N, seed):
    """Host tensors of one batch: unit-ball clouds, per-level features ~N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    d = torch.randn(B, N, 3, generator=g)
    xyz = (d / d.norm(dim=2, keepdim=True) * torch.rand(B, N, 1, generator=g) ** (1.0 / 3.0)).contiguous()
    n_in = [N] + LEVELS["npoint"][:-1]
    sa_feat = [torch.randn(B, c, n, generator=g) for c, n in zip(LEVELS["channels"], n_in)]
    fp_feat = [torch.randn(B, c, m, generator=g) for c, m in zip(LEVELS["channels"], LEVELS["npoint"])]
    return xyz, sa_feat, fp_feat


# ------------------------------------------------------------------ B200 arm: the pipeline

class Pipeline:
    """SA + FP stack on one GPU, three streams:
      s_fps  : the FPS chain (latency-bound launches on at most 128 of the 148 SMs) and the
               gathers of the sampled centres;
      s_geo  : everything else that only needs coordinates (ball query, three_nn, weights),
               level by level behind the FPS events;
      s_feat : the feature work (grouping and interpolation, forward and backward) behind
               the s_geo events, one sub-stream per level (the levels' feature kernels are
               independent of one another), joined on s_feat.
    With pipelined=True consecutive steps are not joined: the geometry of step i+1 (which
    depends on nothing but its input coordinates) runs while the feature work of step i is
    still in flight, as it would behind a prefetching data loader."""

    def __init__(self, dev, B, N, seed):
        import torch_points_kernels_b200 as tpk

        self.tpk = tpk
        self.dev = dev
        self.B, self.N = B, N
        # two FPS streams, used by alternate steps: the chain is latency-bound and leaves the SMs
        # mostly idle, so the chains of two consecutive steps can run side by side
        # High priority: a sampling kernel that becomes ready gets the next free SMs instead of
        # queueing behind the thousands of CTAs of the feature kernels (every later level waits for it)
        # (measured: 9114 against 9024 clouds/s)
        self.s_fps_pair = [torch.cuda.Stream(dev, priority=-1), torch.cuda.Stream(dev, priority=-1)]
        self.s_fps = self.s_fps_pair[0]
        self.nstep = 0
        self.s_geo = torch.cuda.Stream(dev)
        self.s_feat = torch.cuda.Stream(dev)
        # the feature kernels of the four levels do not depend on one another: one stream each,
        # joined on s_feat
        self.s_feat_level = [torch.cuda.Stream(dev) for _ in range(4)]
        self.s_copy = torch.cuda.Stream(dev)
        g = torch.Generator(device=dev).manual_seed(seed + 7)
        # upstream gradients: produced on the device by the layers above in a real model
        n_in = [N] + LEVELS["npoint"][:-1]
        self.g_grouped = [torch.randn(B, c, m, LEVELS["nsample"], device=dev, generator=g)
                          for c, m in zip(LEVELS["channels"], LEVELS["npoint"])]
        self.g_up = [torch.randn(B, c, n, device=dev, generator=g) for c, n in zip(LEVELS["channels"], n_in)]
        self.keep = None

    def step(self, xyz, sa_feat, fp_feat, overlap=True, timers=None, pipelined=False, ready=None):
        """xyz (B,N,3), sa_feat[l] (B,C_l,N_l), fp_feat[l] (B,C_l,M_l) on the device.
        Returns (fps indices of every level, gradients of the SA features, of the FP
        features, event recorded when the step's last kernel has been enqueued).
        `ready`: event after which the inputs may be read (pipelined mode)."""
        tpk = self.tpk
        cur = torch.cuda.current_stream(self.dev)
        self.s_fps = self.s_fps_pair[self.nstep & 1] if pipelined else self.s_fps_pair[0]
        self.nstep += 1
        s_fps = self.s_fps if overlap else cur
        s_geo = self.s_geo if overlap else cur
        s_feat = self.s_feat if overlap else cur
        if overlap:
            for st in (s_fps, s_geo, s_feat):
                if pipelined:
                    if ready is not None:
                        st.wait_event(ready)
                else:
                    st.wait_stream(cur)

        def timed(name, fn):
            if timers is None:
                return fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(torch.cuda.current_stream(self.dev))
            out = fn()
            e1.record(torch.cuda.current_stream(self.dev))
            timers.setdefault(name, []).append((e0, e1))
            return out

        def hand_over(t, *streams):
            # the caching allocator must not recycle t while another stream still reads it;
            # under graph capture every intermediate is simply kept alive for the whole step
            if self.keep is not None:
                self.keep.append(t)
            elif overlap:
                for st in streams:
                    t.record_stream(st)
            return t

        def level_stream(l):
            # Under graph capture the feature kernels of each level get a branch of their own.
            # Launched eagerly they share s_feat: tensors allocated on four more streams make
            # the caching allocator grow four more pools, which costs more than the overlap gives.
            if not overlap:
                return cur
            return self.s_feat_level[l] if self.keep is not None else s_feat

        pts = [xyz]
        fps_idx, fps_ready = [], []
        with torch.cuda.stream(s_fps):
            for l, m in enumerate(LEVELS["npoint"]):
                # indices and the sampled coordinates from one library call
                idx, centres = timed("fps_l%d" % (l + 1), lambda: tpk.furthest_point_sample(pts[l], m, return_xyz=True))
                fps_idx.append(hand_over(idx, cur))
                pts.append(hand_over(centres, s_geo))
                ev = torch.cuda.Event()
                ev.record(s_fps)
                fps_ready.append(ev)

        geo, geo_ready = [], []
        with torch.cuda.stream(s_geo):
            for l in range(4):
                if overlap:
                    s_geo.wait_event(fps_ready[l])
                r, ns = LEVELS["radius"][l], LEVELS["nsample"]
                nbr, _ = timed("ball_query_l%d" % (l + 1),
                               lambda: tpk.ball_query(r, ns, pts[l], pts[l + 1], mode="dense"))
                # feature propagation of this level: from its centres back to its input points
                dist, idx3 = timed("three_nn_l%d" % (l + 1), lambda: tpk.three_nn(pts[l], pts[l + 1]))
                w = 1.0 / (dist + 1e-8)
                w = (w / w.sum(dim=2, keepdim=True)).contiguous()
                s_lvl = level_stream(l)
                geo.append((hand_over(nbr, s_lvl), hand_over(idx3, s_lvl), hand_over(w, s_lvl)))
                ev = torch.cuda.Event()
                ev.record(s_geo)
                geo_ready.append(ev)

        grads_sa, grads_fp = [], []
        for l in range(4):
            s_lvl = level_stream(l)
            with torch.cuda.stream(s_lvl):
                if overlap:
                    if s_lvl is not s_feat:
                        s_lvl.wait_stream(s_feat)  # the inputs' readiness, as s_feat saw it at the start of the step
                    s_lvl.wait_event(geo_ready[l])
                nbr, idx3, w = geo[l]
                f = sa_feat[l].requires_grad_(True)
                grouped = timed("grouping_fwd_l%d" % (l + 1), lambda: tpk.grouping_operation(f, nbr))
                timed("grouping_bwd_l%d" % (l + 1), lambda: grouped.backward(self.g_grouped[l]))
                grads_sa.append(hand_over(f.grad, cur, s_feat))
                f.grad = None
                ff = fp_feat[l].requires_grad_(True)
                up = timed("interp_fwd_l%d" % (l + 1), lambda: tpk.three_interpolate(ff, idx3, w))
                timed("interp_bwd_l%d" % (l + 1), lambda: up.backward(self.g_up[l]))
                grads_fp.append(hand_over(ff.grad, cur, s_feat))
                ff.grad = None
        with torch.cuda.stream(s_feat):
            if overlap and self.keep is not None:
                for st in self.s_feat_level:
                    s_feat.wait_stream(st)
            done = torch.cuda.Event()
            done.record(s_feat)
        if overlap and not pipelined:
            cur.wait_stream(s_fps)
            cur.wait_stream(s_geo)
            cur.wait_stream(s_feat)
        return fps_idx, grads_sa, grads_fp, done


# ------------------------------------------------ the reference's CUDA build, same inputs

def load_reference_cuda():
    """The reference's CUDA extension compiled for sm_100a from its own sources
    (oracle/_ref/points_cuda.so), or (None, reason)."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "points_cuda.so")):
        return None, "oracle/_ref/points_cuda.so has not been built"
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    try:
        import points_cuda

        return points_cuda, None
    except Exception as e:
        return None, "points_cuda.so does not load: %s" % str(e).splitlines()[0][:160]


class RefCudaPipeline:
    """The same SA + FP stack through the reference's own CUDA kernels and launch shapes
    (grouping = torch.gather on the expanded index and its autograd, as in
    torch_points_kernels/torchpoints.py:143-146).  Every op runs on the current stream."""

    def __init__(self, ref, dev, xyz, sa, fp, g_grouped, g_up):
        self.ref, self.dev = ref, dev
        self.xyz, self.sa, self.fp, self.g_grouped, self.g_up = xyz, sa, fp, g_grouped, g_up

    def step(self, times=None):
        ref, B = self.ref, self.xyz.shape[0]

        def t(name, fn):
            if times is None:
                return fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn()
            e1.record()
            times.setdefault(name, []).append((e0, e1))
            return r

        pts = [self.xyz]
        fps_idx, grads_sa, grads_fp = [], [], []
        for l, m in enumerate(LEVELS["npoint"]):
            idx = t("fps_l%d" % (l + 1), lambda: ref.furthest_point_sampling(pts[l], m))
            fps_idx.append(idx)
            centres = torch.gather(pts[l], 1, idx.long().unsqueeze(-1).expand(-1, -1, 3)).contiguous()
            pts.append(centres)
            nbr, _ = t("ball_query_l%d" % (l + 1),
                       lambda: ref.ball_query_dense(centres, pts[l], LEVELS["radius"][l], LEVELS["nsample"]))
            f = self.sa[l].detach().requires_grad_(True)

            def group():
                all_idx = nbr.reshape(B, -1).unsqueeze(1).repeat(1, f.shape[1], 1)
                return f.gather(2, all_idx).reshape(B, f.shape[1], nbr.shape[1], nbr.shape[2])

            grouped = t("grouping_fwd_l%d" % (l + 1), group)
            t("grouping_bwd_l%d" % (l + 1), lambda: grouped.backward(self.g_grouped[l]))
            grads_sa.append(f.grad)
            d2, idx3 = t("three_nn_l%d" % (l + 1), lambda: ref.three_nn(pts[l], centres))
            dist = torch.sqrt(d2)
            w = 1.0 / (dist + 1e-8)
            w = (w / w.sum(dim=2, keepdim=True)).contiguous()
            t("interp_fwd_l%d" % (l + 1), lambda: ref.three_interpolate(self.fp[l], idx3, w))
            grads_fp.append(t("interp_bwd_l%d" % (l + 1),
                              lambda: ref.three_interpolate_grad(self.g_up[l], idx3, w, self.fp[l].shape[2])))
        return fps_idx, grads_sa, grads_fp


def time_reference_cuda(ref, dev, dev_in, split, pipe, steps, in_flight):
    """The reference CUDA build on the same device-resident inputs: one step after the other
    (compare with ms_per_step_isolated) and `in_flight` steps at a time on as many streams
    (compare with ms_per_step), CUDA events around the whole run."""
    xyz, sa, fp = split([t.detach() for t in dev_in])
    rp = RefCudaPipeline(ref, dev, xyz, sa, fp, pipe.g_grouped, pipe.g_up)
    rp.step()
    torch.cuda.synchronize(dev)
    times = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        rp.step(times)
    e1.record()
    torch.cuda.synchronize(dev)
    ms_iso = e0.elapsed_time(e1) / steps
    cur = torch.cuda.current_stream(dev)
    streams = [torch.cuda.Stream(dev) for _ in range(in_flight)]
    rounds = max(2, (steps + in_flight - 1) // in_flight)
    for st in streams:
        st.wait_stream(cur)
    # one untimed step per stream: the allocator's pool of every stream is filled before the clock
    # starts (without it the number swings between 73 and 118 ms per step)
    for st in streams:
        with torch.cuda.stream(st):
            rp.step()
    for st in streams:
        cur.wait_stream(st)
    torch.cuda.synchronize(dev)
    for st in streams:
        st.wait_stream(cur)
    e0.record()
    for _ in range(rounds):
        for st in streams:
            with torch.cuda.stream(st):
                rp.step()
    for st in streams:
        cur.wait_stream(st)
    e1.record()
    torch.cuda.synchronize(dev)
    ms_fly = e0.elapsed_time(e1) / (rounds * in_flight)
    return {"kind": "reference CUDA extension, rebuilt for sm_100a from the reference sources, same inputs",
            "ms_per_step_isolated": round(ms_iso, 3), "steps_isolated": steps,
            "ms_per_step_in_flight": round(ms_fly, 3), "streams_in_flight": in_flight, "steps_in_flight": rounds * in_flight,
            "clouds_per_s_isolated": round(xyz.shape[0] / (ms_iso * 1e-3), 2),
            "clouds_per_s_in_flight": round(xyz.shape[0] / (ms_fly * 1e-3), 2),
            "kernels_ms": {k: round(sorted(a.elapsed_time(b) for a, b in v)[len(v) // 2], 4)
                           for k, v in sorted(times.items())}}, rp


def verify_against_reference_cuda(rp, fps_idx, g_sa, g_fp):
    """Outside every timed region: the sampled indices of all four levels must equal the
    reference CUDA build's, and every gradient tensor's L2 norm must agree to 1e-4 relative
    (atomic accumulation order differs).  Returns (verified, detail)."""
    r_idx, r_sa, r_fp = rp.step()
    torch.cuda.synchronize()
    detail = {}
    ok = True
    for l in range(4):
        same = bool(torch.equal(fps_idx[l], r_idx[l]))
        detail["fps_idx_l%d" % (l + 1)] = same
        ok &= same
    worst = 0.0
    for mine, theirs in zip(list(g_sa) + list(g_fp), list(r_sa) + list(r_fp)):
        a, b = float(mine.double().norm()), float(theirs.double().norm())
        worst = max(worst, abs(a - b) / max(b, 1e-30))
    detail["grad_norm_max_rel_diff"] = float("%.3g" % worst)
    ok &= worst <= 1e-4
    return ok, detail


def graph_time(fn, dev, inner=10, reps=3):
    """Device time of one call of fn: `inner` calls captured into one CUDA graph and replayed,
    so that neither Python nor launch gaps are inside the measurement."""
    fn()
    torch.cuda.synchronize(dev)
    side = torch.cuda.Stream(dev)
    graph = torch.cuda.CUDAGraph()
    keep = []
    with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
        for _ in range(inner):
            keep.append(fn())
    graph.replay()
    torch.cuda.synchronize(dev)
    best = None
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / inner
        best = ms if best is None else min(best, ms)
    del keep
    return best


def grid_candidates(points, queries, h_min, max_dim):
    """Mean number of candidate points in the 3x3x3 block of grid cells around a query, for a
    uniform grid over each cloud's bounding box with cells max(h_min, extent / max_dim) wide:
    the grid the shared-memory search kernels build.  points (B,N,3), queries (B,M,3)."""
    B = points.shape[0]
    lo = points.amin(dim=1, keepdim=True)
    ext = (points.amax(dim=1, keepdim=True) - lo).amax(dim=2, keepdim=True)
    h = torch.clamp(ext / max_dim, min=h_min)
    d = int(max_dim)
    cp = torch.clamp(((points - lo) / h).long(), 0, d - 1)
    cq = torch.clamp(((queries - lo) / h).long(), 0, d - 1)
    flat = (cp[..., 2] * d + cp[..., 1]) * d + cp[..., 0]
    hist = torch.zeros(B, d * d * d, device=points.device)
    hist.scatter_add_(1, flat, torch.ones_like(flat, dtype=torch.float32))
    box = torch.nn.functional.avg_pool3d(hist.view(B, 1, d, d, d), 3, stride=1, padding=1, count_include_pad=True) * 27.0
    fq = (cq[..., 2] * d + cq[..., 1]) * d + cq[..., 0]
    return float(box.view(B, -1).gather(1, fq).mean())


def per_kernel_times(pipe, dev, ins):
    """Device time of every op of the step at its pipeline shape (graph replay, see graph_time)
    and, for the grid searches, (candidates per query, queries per launch)."""
    tpk = pipe.tpk
    xyz, sa_feat, fp_feat = ins
    kms, cand = {}, {}
    pts = [xyz]
    ns = LEVELS["nsample"]
    for l, m in enumerate(LEVELS["npoint"]):
        tag = "_l%d" % (l + 1)
        r = LEVELS["radius"][l]
        src = pts[l]
        kms["fps" + tag] = graph_time(lambda: tpk.furthest_point_sample(src, m, return_xyz=True), dev, inner=3)
        _, centres = tpk.furthest_point_sample(src, m, return_xyz=True)
        pts.append(centres)
        kms["ball_query" + tag] = graph_time(lambda: tpk.ball_query(r, ns, src, centres, mode="dense"), dev)
        kms["three_nn" + tag] = graph_time(lambda: tpk.three_nn(src, centres), dev)
        nbr, _ = tpk.ball_query(r, ns, src, centres, mode="dense")
        dist, idx3 = tpk.three_nn(src, centres)
        w = 1.0 / (dist + 1e-8)
        w = (w / w.sum(dim=2, keepdim=True)).contiguous()
        f, ff = sa_feat[l].detach(), fp_feat[l].detach()
        kms["grouping_fwd" + tag] = graph_time(lambda: tpk.grouping_operation(f, nbr), dev)
        kms["interp_fwd" + tag] = graph_time(lambda: tpk.three_interpolate(ff, idx3, w), dev)
        # the backward kernels alone, through the same C entry points autograd calls
        n = f.shape[2]
        gg, gu = pipe.g_grouped[l], pipe.g_up[l]
        kms["grouping_bwd" + tag] = graph_time(lambda: tpk.torchpoints.grouping_backward(gg, nbr, n), dev)
        kms["interp_bwd" + tag] = graph_time(lambda: tpk.torchpoints.three_interpolate_backward(gu, idx3, w, m), dev)
        # the fused set-abstraction grouping (centres + ball query + relative coordinates + features
        # in one call) beside the sequence a caller of the separate ops runs for the same tensor
        fidx = tpk.furthest_point_sample(src, m)
        kms["sa_group" + tag] = graph_time(lambda: tpk.sa_group(src, f, fidx, r, ns), dev)

        def unfused():
            c_xyz = torch.gather(src, 1, fidx.long().unsqueeze(-1).expand(-1, -1, 3)).contiguous()
            nb, _ = tpk.ball_query(r, ns, src, c_xyz, mode="dense")
            rel = tpk.grouping_operation(src.transpose(1, 2).contiguous(), nb) - c_xyz.transpose(1, 2).unsqueeze(-1)
            return torch.cat([rel, tpk.grouping_operation(f, nb)], dim=1)

        kms["sa_unfused_sequence" + tag] = graph_time(unfused, dev)
        n_in = src.shape[1]
        if n_in >= 1024:  # ball query on the shared-memory grid: cells one radius wide or wider
            cand["ball_query" + tag] = (grid_candidates(src, centres, r, grid_max_dim(n_in)), src.shape[0] * m)
        if 256 <= m <= 8192:  # three_nn on the grid of the known points
            cand["three_nn" + tag] = (grid_candidates(centres, src, 1e-30, grid_max_dim(m)), src.shape[0] * n_in)
    return kms, cand


def grid_max_dim(n, cap=64):
    """Cells per axis the search kernels use for a cloud of n points: about two points per cell."""
    d = 4
    while d < cap and (d + 1) ** 3 * 2 <= n:
        d += 1
    return d



def flat_views(like, dev, pinned):
    """One uint8 buffer (device, or pinned host) and float32 views of it shaped like `like`,
    each starting on a 256-byte boundary."""
    offs, total = [], 0
    for t in like:
        offs.append(total)
        total += (t.numel() * t.element_size() + 255) // 256 * 256
    flat = torch.empty(total, dtype=torch.uint8, pin_memory=True) if pinned else torch.empty(total, dtype=torch.uint8, device=dev)
    views = [flat[o:o + t.numel() * t.element_size()].view(t.dtype).view(t.shape) for o, t in zip(offs, like)]
    return flat, views


def checksums(tensors):
    """One number per gradient tensor for the device-to-host result of a step: the L2 norms,
    computed for all tensors by one multi-tensor kernel."""
    return torch.stack(torch._foreach_norm(list(tensors)))


def _lib_launches():
    from torch_points_kernels_b200 import _lib

    return _lib.kernel_launches()


class GraphedSteps:
    """`nslots` CUDA graphs of one whole step each (all three internal streams captured), replayed
    in turn, each on its own launch stream: no per-kernel host work, and consecutive steps still
    overlap because they are launched on different streams."""

    def __init__(self, pipe, dev, like, split, nslots=3):
        self.slots = []
        for _ in range(nslots):
            # the step's inputs are views of one buffer, so that a step's host-to-device copy is one transfer
            flat, ins = flat_views(like, dev, pinned=False)
            launch = torch.cuda.Stream(dev)
            graph = torch.cuda.CUDAGraph()
            pipe.keep = []
            before = _lib_launches()
            try:
                with torch.cuda.graph(graph, stream=launch, capture_error_mode="thread_local"):
                    fps_idx, g_sa, g_fp, _ = pipe.step(*split([t.detach() for t in ins]))
                    chk = checksums(g_sa + g_fp)
            finally:
                keep, pipe.keep = pipe.keep, None
            # kernels of the library in one step: counted by the library while the step was captured
            self.launches_per_step = _lib_launches() - before
            self.slots.append({"graph": graph, "ins": ins, "flat": flat, "launch": launch, "fps_idx": fps_idx, "chk": chk,
                               "keep": (keep, g_sa, g_fp)})

    def load(self, tensors):
        for slot in self.slots:
            for dst, src in zip(slot["ins"], tensors):
                dst.copy_(src)


def pipeline_work(B, N):
    """Algorithmic bytes (HBM-bound kernels) or FP32-pipe lane operations (search kernels,
    6 per point pair: 3 subtractions, 1 multiply, 2 fused multiply-adds) per launch."""
    n_in = [N] + LEVELS["npoint"][:-1]
    ns = LEVELS["nsample"]
    w = {}
    for l in range(4):
        n, m, c = n_in[l], LEVELS["npoint"][l], LEVELS["channels"][l]
        w["grouping_fwd_l%d" % (l + 1)] = ("hbm", 4 * B * c * m * ns + 8 * B * m * ns + 4 * B * c * n)
        w["grouping_bwd_l%d" % (l + 1)] = ("hbm", 4 * B * c * m * ns + 8 * B * m * ns + 2 * 4 * B * c * n)
        w["interp_fwd_l%d" % (l + 1)] = ("hbm", 4 * B * c * n + 4 * B * c * m + B * n * 3 * 8)
        w["interp_bwd_l%d" % (l + 1)] = ("hbm", 4 * B * c * n + 2 * 4 * B * c * m + B * n * 3 * 8)
        # brute-force-equivalent pairs (what the reference's scans evaluate); the grid searches
        # (three_nn with 256..8192 known points, ball query on 1024+ points) look at a few dozen
        # candidates per query instead, counted separately in run_b200
        w["three_nn_l%d" % (l + 1)] = ("fp32", 6 * B * n * m)
        w["ball_query_l%d" % (l + 1)] = ("fp32", 6 * B * m * n)
        # brute-force-equivalent work: the sorted kernels skip most of it in late rounds
        w["fps_l%d" % (l + 1)] = ("fp32", 6 * B * (m - 1) * n)
    return w


# DRAM bytes (read + write) of one launch of the HBM-bound kernels at the bench's own shape
# (16 clouds), from one-launch ncu captures of dram__bytes_read.sum and dram__bytes_write.sum;
# the commands and figures are in the summaries under profiles/.
NCU_TRAFFIC_BYTES = {
    "grouping_bwd_l1": (16794368 + 0) + (546299904 + 52450304),  # sort kernel + summing kernel
    "grouping_fwd_l1": 84018432 + 476870912,
    "interp_fwd_l1": 23094784 + 9831680,
    "interp_bwd_l1": 73415168 + 2494976,
}


def sample_clocks(stop, path, dev_index):
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    try:
        with open(path, "w") as f:
            p = subprocess.Popen(["nvidia-smi", "-i", str(dev_index), "--query-gpu=" + q,
                                  "--format=csv,noheader,nounits", "-lms", "100"], stdout=f,
                                 stderr=subprocess.DEVNULL)
            stop.wait()
            p.terminate()
            p.wait(timeout=5)
    except Exception:
        pass


def parse_clocks(path):
    sm, mx, reasons = [], 0, set()
    try:
        for line in open(path):
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx = max(mx, float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
    except OSError:
        pass
    sm.sort()
    return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
            "samples": len(sm)}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def bind_near_gpu(dev_index):
    """Moves this process onto the host cores of the NUMA node its GPU hangs off, before any pinned
    buffer is allocated (pages land on the node of the thread that first touches them), so that
    the per-step host-to-device copy does not cross the socket link.  Returns what it did for the
    JSON line; a container that only sees one node's cores is left as it is."""
    try:
        p = torch.cuda.get_device_properties(dev_index)
        pci = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % pci).read())
        if node < 0:
            return {"node": None, "note": "the platform reports no NUMA node for the GPU"}
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        near = cpus & allowed
        if not near:
            return {"node": node, "note": "none of the %d cores this process may use is on that node" % len(allowed)}
        os.sched_setaffinity(0, near)
        return {"node": node, "cores": len(near), "of_allowed": len(allowed)}
    except (OSError, ValueError, AttributeError) as e:
        return {"node": None, "note": "not bound: %s" % e}


def run_b200(args, rank, world, local_rank):
    import torch.distributed as dist

    from torch_points_kernels_b200 import _lib

    _lib.lib()  # fail loudly if the CUDA library is missing
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    host_binding = bind_near_gpu(local_rank)
    B, N = B_CLOUDS, N_POINTS
    xyz_h, sa_h, fp_h = make_inputs(B, N, 2000 + rank)
    host = [xyz_h] + sa_h + fp_h
    pinned_flat, pinned = flat_views(host, None, pinned=True)
    for dst, src in zip(pinned, host):
        dst.copy_(src)
    dev_in = [t.to(dev) for t in host]
    pipe = Pipeline(dev, B, N, 2000 + rank)

    def split(ts):
        return ts[0], list(ts[1:5]), list(ts[5:9])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing (inputs already in HBM); > 1 GB moves per step, far beyond L2
    cur = torch.cuda.current_stream(dev)

    def run_resident(k, pipelined):
        """k steps; pipelined: at most three steps in flight (bounds memory held by the
        allocator for cross-stream tensors), one join at the end."""
        dones = []
        host = 0.0
        for i in range(k):
            if pipelined and i >= 3:
                dones[i - 3].synchronize()
            t0 = time.perf_counter()
            out = pipe.step(*split([t.detach() for t in dev_in]), pipelined=pipelined)
            host += time.perf_counter() - t0
            dones.append(out[3])
        pipe.host_ms = host * 1e3 / max(k, 1)
        if pipelined:
            for st in pipe.s_fps_pair:
                cur.wait_stream(st)
            cur.wait_stream(pipe.s_geo)
            cur.wait_stream(pipe.s_feat)

    run_resident(args.warmup, True)
    torch.cuda.synchronize(dev)
    graphs, graph_error = None, None
    if not args.no_graphs:
        try:
            graphs = GraphedSteps(pipe, dev, dev_in, split, args.in_flight)
            graphs.load(dev_in)
            torch.cuda.synchronize(dev)
        except Exception as e:  # fall back to eager launches, and say so in the JSON line
            graphs = None
            graph_error = "%s: %s" % (type(e).__name__, str(e).splitlines()[0][:200])
            torch.cuda.synchronize(dev)

    def run_graphs(k):
        t0 = time.perf_counter()
        for i in range(k):
            slot = graphs.slots[i % len(graphs.slots)]
            with torch.cuda.stream(slot["launch"]):
                slot["graph"].replay()
        pipe.host_ms = (time.perf_counter() - t0) * 1e3 / max(k, 1)
        for slot in graphs.slots:
            cur.wait_stream(slot["launch"])

    if graphs is not None:
        run_graphs(args.warmup)
        torch.cuda.synchronize(dev)
    stop = threading.Event()
    clock_file = os.path.join(tempfile.gettempdir(), "tpk_clocks_%d.csv" % rank)
    sampler = threading.Thread(target=sample_clocks, args=(stop, clock_file, local_rank), daemon=True)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed_region(body):
        """EXACTLY args.steps steps between a barrier + synchronize on both sides, CUDA events on
        the current stream, maximum over ranks."""
        barrier()
        e0.record()
        body()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    def repeated(body, min_total_ms, max_reps):
        """The timed region again and again until the repetitions cover min_total_ms (so that the
        clock sampler sees the GPU under load); every rank derives the same count from the
        rank-reduced time of the first one.  Returns the sorted per-repetition times."""
        first = timed_region(body)
        reps = int(min(max_reps, max(3, -(-min_total_ms // max(first, 1e-3)))))
        return sorted([first] + [timed_region(body) for _ in range(reps - 1)])

    launches_before = _lib.kernel_launches()

    def resident_body():
        if graphs is not None:
            for slot in graphs.slots:
                slot["launch"].wait_stream(cur)
            run_graphs(args.steps)
        else:
            run_resident(args.steps, True)

    reps_total = repeated(resident_body, args.min_seconds * 1e3, 400)
    ms_total = reps_total[len(reps_total) // 2]
    if graphs is not None:
        launches = graphs.launches_per_step * args.steps  # replays are not seen by the library's counter
    else:
        launches = (_lib.kernel_launches() - launches_before) // len(reps_total)
    host_ms = pipe.host_ms

    # the same without overlap between consecutive steps (latency of one isolated step)
    def isolated_body():
        if graphs is not None:
            slot = graphs.slots[0]
            slot["launch"].wait_stream(cur)
            with torch.cuda.stream(slot["launch"]):
                for _ in range(args.steps):
                    slot["graph"].replay()
            cur.wait_stream(slot["launch"])
        else:
            run_resident(args.steps, False)

    reps_isolated = repeated(isolated_body, 250.0, 20)
    ms_isolated = reps_isolated[len(reps_isolated) // 2]

    # ---- end to end: pinned host inputs copied in on a copy stream, results (sampled indices
    # and one checksum per gradient tensor) copied out to pinned host buffers, every step
    out_bufs = [[torch.empty((B, m), dtype=torch.int32).pin_memory() for m in LEVELS["npoint"]] +
                [torch.empty((8,), dtype=torch.float32).pin_memory()] for _ in range(max(3, args.in_flight))]

    def run_e2e(k):
        dones = []
        for i in range(k):
            if i >= 3:
                dones[i - 3].synchronize()
            with torch.cuda.stream(pipe.s_copy):
                ins = [p.to(dev, non_blocking=True) for p in pinned]
                ready = torch.cuda.Event()
                ready.record(pipe.s_copy)
            for st in pipe.s_fps_pair:
                ins[0].record_stream(st)
            ins[0].record_stream(pipe.s_geo)
            for t in ins[1:]:
                t.record_stream(pipe.s_feat)
                for st in pipe.s_feat_level:
                    t.record_stream(st)
            fps_idx, g_sa, g_fp, _ = pipe.step(*split(ins), pipelined=True, ready=ready)
            bufs = out_bufs[i % 3]
            with torch.cuda.stream(pipe.s_feat):
                for ev_src, dst in zip(fps_idx, bufs[:4]):
                    ev_src.record_stream(pipe.s_feat)
                pipe.s_feat.wait_stream(pipe.s_fps)
                for src, dst in zip(fps_idx, bufs[:4]):
                    dst.copy_(src, non_blocking=True)
                chk = checksums(g_sa + g_fp)
                bufs[4].copy_(chk, non_blocking=True)
                done = torch.cuda.Event()
                done.record(pipe.s_feat)
            dones.append(done)
        cur.wait_stream(pipe.s_copy)
        for st in pipe.s_fps_pair:
            cur.wait_stream(st)
        cur.wait_stream(pipe.s_geo)
        cur.wait_stream(pipe.s_feat)
        return out_bufs[(k - 1) % 3]

    def run_e2e_graphs(k):
        for slot in graphs.slots:
            slot["launch"].wait_stream(cur)
        for i in range(k):
            slot = graphs.slots[i % len(graphs.slots)]
            bufs = out_bufs[i % len(graphs.slots)]
            with torch.cuda.stream(slot["launch"]):
                slot["flat"].copy_(pinned_flat, non_blocking=True)  # all inputs of the step, one transfer
                slot["graph"].replay()
                for src, dst in zip(slot["fps_idx"], bufs[:4]):
                    dst.copy_(src, non_blocking=True)
                bufs[4].copy_(slot["chk"], non_blocking=True)
        for slot in graphs.slots:
            cur.wait_stream(slot["launch"])
        return out_bufs[(k - 1) % len(graphs.slots)]

    if graphs is not None:
        run_e2e = run_e2e_graphs
    run_e2e(max(2, args.warmup // 2))
    res_box = []
    reps_e2e = repeated(lambda: res_box.append(run_e2e(args.steps)), args.min_seconds * 1e3, 400)
    ms_e2e = reps_e2e[len(reps_e2e) // 2]
    res = res_box[-1]

    # ceiling of the end-to-end number set by the host link alone: the same pinned buffer copied
    # to the device once per step on the same launch streams, no kernels
    h2d_targets = [slot["flat"] for slot in graphs.slots] if graphs is not None else [torch.empty_like(pinned_flat, device=dev)]
    h2d_streams = [slot["launch"] for slot in graphs.slots] if graphs is not None else [pipe.s_copy]

    def h2d_body():
        for st in h2d_streams:
            st.wait_stream(cur)
        for i in range(args.steps):
            with torch.cuda.stream(h2d_streams[i % len(h2d_streams)]):
                h2d_targets[i % len(h2d_targets)].copy_(pinned_flat, non_blocking=True)
        for st in h2d_streams:
            cur.wait_stream(st)

    reps_h2d = repeated(h2d_body, 250.0, 20)
    ms_h2d = reps_h2d[len(reps_h2d) // 2]
    if graphs is not None:
        graphs.load(dev_in)  # the copies above overwrote the slots' inputs with the same values; keep them defined
        torch.cuda.synchronize(dev)
    h2d = sum(t.numel() * t.element_size() for t in pinned)  # payload (the transfer pads each tensor to 256 bytes)
    d2h = sum(t.numel() * t.element_size() for t in res)
    if rank == 0:
        stop.set()
        sampler.join(timeout=10)
    clocks = parse_clocks(clock_file) if rank == 0 else {}

    if rank != 0:
        return

    # ---- per-kernel device times: every op of the step alone, ten calls captured into one CUDA
    # graph and replayed (no Python, no launch gaps inside the measurement)
    kms, cand = per_kernel_times(pipe, dev, split([t.detach() for t in dev_in]))

    # ---- outside every timed region: the step's results against the reference's CUDA build, and
    # that build's own time on the same inputs (the target the speed-up is defined against)
    verified, verify_detail, ref_cuda = None, None, None
    ref_mod, ref_err = load_reference_cuda()
    if world == 1 and not args.no_reference_cuda:
        if ref_mod is None:
            ref_cuda = {"unavailable": ref_err}
        else:
            ref_cuda, rp = time_reference_cuda(ref_mod, dev, dev_in, split, pipe, 10, args.in_flight)
            if graphs is not None:
                slot = graphs.slots[0]
                slot["graph"].replay()
                torch.cuda.synchronize(dev)
                verified, verify_detail = verify_against_reference_cuda(rp, slot["fps_idx"], slot["keep"][1], slot["keep"][2])
            else:
                out = pipe.step(*split([t.detach() for t in dev_in]))
                torch.cuda.synchronize(dev)
                verified, verify_detail = verify_against_reference_cuda(rp, out[0], out[1], out[2])
            del rp
    hbm_peak, peak_kind = measured_peaks()
    work = pipeline_work(B, N)
    sm_mhz = clocks.get("sm_mhz") or 1965.0
    fp32_peak_lane_ops = 148 * 128 * sm_mhz * 1e6  # lane-ops / s at the sampled clock
    kernels = {}
    fused = {}
    for l in range(1, 5):
        a, b2 = kms.pop("sa_group_l%d" % l), kms.pop("sa_unfused_sequence_l%d" % l)
        fused["l%d" % l] = {"sa_group_ms": round(a, 4), "unfused_sequence_ms": round(b2, 4),
                            "ball_query_plus_grouping_fwd_ms": round(kms["ball_query_l%d" % l] + kms["grouping_fwd_l%d" % l], 4)}
    fused["what"] = ("sa_group = centres + ball query + relative coordinates + features written as one (B,3+C,M,ns) "
                     "tensor; unfused_sequence = gather, ball_query, two grouping_operations, subtraction and cat for the "
                     "same tensor; the third figure is ball query + feature grouping alone (no coordinates, no cat)")
    for name, ms in sorted(kms.items()):
        kind, amount = work[name]
        entry = {"ms": round(ms, 4), "bound": kind}
        if kind == "hbm":
            entry["achieved_gbs"] = round(amount / ms / 1e6, 1)
            entry["frac"] = round(amount / ms / 1e6 / hbm_peak, 4)
        else:
            # FP32 pipe: 6 lane-ops per (query, candidate) pair over the time taken, against
            # 148 SMs x 128 lanes at the sampled clock.  `frac` counts the candidates the grid
            # search examines (3x3x3 cell block, a lower bound for three_nn, whose search may
            # grow); `frac_brute_force` counts every pair of the cloud, i.e. what the
            # reference's scan evaluates - above 1 where the grid skips most of them.
            entry["frac_brute_force"] = round(amount / (ms * 1e-3) / fp32_peak_lane_ops, 4)
            if name in cand:
                entry["candidates_per_query"] = round(cand[name][0], 1)
                entry["lane_ops"] = int(6 * cand[name][0] * cand[name][1])
                entry["frac"] = round(entry["lane_ops"] / (ms * 1e-3) / fp32_peak_lane_ops, 4)
            else:
                entry["lane_ops"] = amount
                entry["frac"] = entry["frac_brute_force"]
        kernels[name] = entry
    dom = max((k for k in kernels if kernels[k]["bound"] == "hbm"), key=lambda k: kms[k])
    roof = {"kernel": dom, "bound": "hbm", "achieved": kernels[dom]["achieved_gbs"], "peak": hbm_peak,
            "peak_source": peak_kind, "unit": "GB/s", "frac": kernels[dom]["frac"], "traffic": NCU_TRAFFIC_BYTES.get(dom),
            "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at this shape "
                              "(B=16), see profiles/" if dom in NCU_TRAFFIC_BYTES else None,
            "algorithmic_bytes": work[dom][1],
            "time_dominant_kernel": max(kms, key=kms.get)}
    clouds = B * world
    line = {
        "metric": METRIC, "value": round(clouds * args.steps / (ms_total * 1e-3), 2), "unit": "clouds/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_total / args.steps, 4),
        "repetitions": len(reps_total),
        "timed_region_ms": {"median": round(ms_total, 3), "min": round(reps_total[0], 3), "max": round(reps_total[-1], 3),
                            "total": round(sum(reps_total), 1),
                            "what": "each repetition is one timed region of exactly `steps` steps between barriers; "
                                    "value is steps / the median repetition"},
        "ms_per_step_isolated": round(ms_isolated / args.steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "pointnet2_ssg_sa_fp_stack fwd+bwd, B=16 clouds x N=16384 per GPU, "
                               "npoint 4096/1024/256/64, radius 0.1/0.2/0.4/0.8, nsample 32, C 64/128/256/512",
                   "clouds_per_gpu": B, "points_per_cloud": N, "parallelism": "batch-sharded x%d" % world,
                   "l2": "each step moves > 1 GB (inputs larger than L2), no explicit flush",
                   "steps_in_flight": "up to %d (one CUDA graph each): the geometry kernels of a step (FPS, ball "
                                      "query, three_nn; they depend on its coordinates only) overlap the feature "
                                      "kernels of the steps before; ms_per_step_isolated is the same step with a "
                                      "join after every step; the FPS chain of one step (sum of kernels.fps_l*) "
                                      "runs beside the other kernels of the steps around it"
                                      % (args.in_flight if graphs is not None else 3)},
        "e2e": {"value": round(clouds * args.steps / (ms_e2e * 1e-3), 2), "unit": "clouds/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(ms_e2e / args.steps, 4),
                "repetitions": len(reps_e2e),
                "h2d_only_ms": round(ms_h2d / args.steps, 4),
                "h2d_only_gbs": round(pinned_flat.numel() / (ms_h2d / args.steps) / 1e6, 1),
                "h2d_only_what": "the step's pinned input buffer copied to the device once per step on the same "
                                 "streams, no kernels: the floor the host link sets for e2e.ms_per_step",
                "host_binding": host_binding},
        "gpu_launches": launches,
        "host_enqueue_ms_per_step": round(host_ms, 3),
        "launch_mode": "cuda graphs (one per step, %d in rotation)" % args.in_flight if graphs is not None else "eager",
        "graph_error": graph_error,
        "clocks": clocks,
        "roofline": roof,
        "kernels": kernels,
    }
    line["fused_sa_group"] = fused
    line["verified"] = verified
    line["verified_detail"] = verify_detail
    if ref_cuda is not None:
        if "ms_per_step_isolated" in ref_cuda:
            ref_cuda["speedup_isolated"] = round(ref_cuda["ms_per_step_isolated"] / (ms_isolated / args.steps), 2)
            ref_cuda["speedup_in_flight"] = round(ref_cuda["ms_per_step_in_flight"] / (ms_total / args.steps), 2)
            ref_cuda["speedup_e2e_vs_isolated"] = round(ref_cuda["ms_per_step_isolated"] / (ms_e2e / args.steps), 2)
        line["reference_cuda"] = ref_cuda
    if world == 1 and not args.no_chamfer:
        line["chamfer"] = chamfer_numbers(dev, ref_mod, 10, 3, cpu=not args.no_cpu_baseline)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_sample()
    print(json.dumps(line), flush=True)


# ------------------------------------------------- reference arm / CPU baseline (host cores)

def load_reference_cpu():
    """The reference's CPU extension built from its own sources, or None."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if os.path.exists(os.path.join(ref_dir, "points_cpu.so")):
        sys.path.insert(0, ref_dir)
        try:
            import points_cpu

            return points_cpu
        except Exception:
            return None
    return None


def cpu_pipeline(xyz, sa_feat, fp_feat, g_grouped, g_up, ref):
    """The same stack on CPU tensors.  With `ref`: the reference's CPU functions (FPS from
    cpu/src/fps.cpp with a fixed start, nanoflann ball query and kNN, accessor-loop
    interpolation, torch.gather grouping as in torchpoints.py:143-146).  Without: the oracle."""
    pts = [xyz]
    if ref is None:
        from oracle import oracle as orc
    for l, m in enumerate(LEVELS["npoint"]):
        r, ns = LEVELS["radius"][l], LEVELS["nsample"]
        if ref is not None:
            idx = ref.fps(pts[l], m, False)
            centres = torch.gather(pts[l], 1, idx.unsqueeze(-1).expand(-1, -1, 3)).contiguous()
            nbr, _ = ref.dense_ball_query(centres, pts[l], r, ns, 0, False)
            f = sa_feat[l].requires_grad_(True)
            all_idx = nbr.reshape(nbr.shape[0], -1).unsqueeze(1).repeat(1, f.shape[1], 1)
            grouped = f.gather(2, all_idx).reshape(nbr.shape[0], f.shape[1], nbr.shape[1], nbr.shape[2])
            grouped.backward(g_grouped[l])
            idx3, d2 = ref.dense_knn(centres, pts[l], 3)
            dist = torch.sqrt(d2)
            w = 1.0 / (dist + 1e-8)
            w = (w / w.sum(dim=2, keepdim=True)).contiguous()
            up = ref.knn_interpolate(fp_feat[l], idx3, w)
            ref.knn_interpolate_grad(g_up[l].contiguous(), idx3, w, fp_feat[l].shape[2])
            del up
        else:
            idx = torch.from_numpy(orc.fps(pts[l], m)).long()
            centres = torch.gather(pts[l], 1, idx.unsqueeze(-1).expand(-1, -1, 3)).contiguous()
            nbr, _ = orc.ball_query_dense(r, ns, pts[l], centres)
            orc.grouping(sa_feat[l], nbr)
            orc.grouping_grad(g_grouped[l], nbr, pts[l].shape[1])
            d2, idx3 = orc.three_nn(pts[l], centres)
            dist = torch.sqrt(torch.from_numpy(d2))
            w = 1.0 / (dist + 1e-8)
            w = (w / w.sum(dim=2, keepdim=True)).contiguous()
            orc.three_interpolate(fp_feat[l], idx3, w)
            orc.three_interpolate_grad(g_up[l], idx3, w, fp_feat[l].shape[2])
        pts.append(centres)


def cpu_inputs(sample_clouds):
    xyz, sa, fp = make_inputs(sample_clouds, N_POINTS, 2000)
    g = torch.Generator().manual_seed(9)
    n_in = [N_POINTS] + LEVELS["npoint"][:-1]
    g_grouped = [torch.randn(sample_clouds, c, m, LEVELS["nsample"], generator=g)
                 for c, m in zip(LEVELS["channels"], LEVELS["npoint"])]
    g_up = [torch.randn(sample_clouds, c, n, generator=g) for c, n in zip(LEVELS["channels"], n_in)]
    return xyz, sa, fp, g_grouped, g_up


def cpu_baseline_sample(sample_clouds=16):
    ref = load_reference_cpu()
    ins = cpu_inputs(sample_clouds)
    t0 = time.perf_counter()
    cpu_pipeline(*ins, ref)
    dt = time.perf_counter() - t0
    return {"value": round(sample_clouds / dt, 4), "unit": "clouds/s", "cores": torch.get_num_threads(),
            "kind": "reference" if ref is not None else "port",
            "sample": "%d clouds = one full step (N=16384, all four SA/FP levels, fwd+bwd), one pass, %.1f s"
                      % (sample_clouds, dt)}


def run_reference(args, rank, world):
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to its workers; this arm is the one CPU process of the
    # run and uses every host core torch can
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    ref = load_reference_cpu()
    sample = 1
    ins = cpu_inputs(sample)
    for _ in range(min(args.warmup, 1)):  # one warm-up pass is enough for a deterministic CPU loop
        cpu_pipeline(*ins, ref)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pipeline(*ins, ref)
    dt = time.perf_counter() - t0
    v = round(sample * args.steps / dt, 4)
    kind = "reference" if ref is not None else "port"
    desc = "%d of the 16 clouds of one step per timed step (N=16384, all four SA/FP levels, fwd+bwd)" % sample
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "clouds/s", "n_gpus": world,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": round(dt / args.steps * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "pointnet2_ssg_sa_fp_stack fwd+bwd, N=16384, npoint 4096/1024/256/64, "
                               "radius 0.1/0.2/0.4/0.8, nsample 32, C 64/128/256/512; CPU sample of %d cloud" % sample},
        "cpu_baseline": {"value": v, "unit": "clouds/s", "cores": torch.get_num_threads(), "kind": kind, "sample": desc},
        "e2e": {"value": v, "unit": "clouds/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def _time_calls(fn, steps, warmup, dev):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) / steps


def chamfer_numbers(dev, ref_mod, steps, warmup, cpu, shapes=((32, 16384), (64, 2048)), lo=0, hi=None):
    """Second leg of the metric: ChamferDistance forward + backward, pairs per second, for pairs
    [lo, hi) of each configuration; beside it the reference's CUDA build on the same inputs and
    (cpu=True) the CPU oracle port on a bounded sample of pairs (the reference has no CPU chamfer)."""
    from torch_points_kernels_b200 import chamfer_dist as cd
    from torch_points_kernels_b200 import synthetic as data

    sm_mhz = 1965.0
    lanes = 148 * 128 * sm_mhz * 1e6
    out = {"metric": "chamfer_pairs_per_s", "unit": "pairs/s", "what": "chamfer_dist(x1, x2).backward(), CUDA events, "
           "%d calls after %d warm-up calls, inputs resident" % (steps, warmup)}
    for B, N in shapes:
        c1, c2 = data.chamfer_pair(B, N, seed=4000)
        c1, c2 = c1[lo:hi], c2[lo:hi]
        nb = c1.shape[0]
        x1, x2 = c1.to(dev).requires_grad_(True), c2.to(dev).requires_grad_(True)

        def fwd_bwd():
            x1.grad = None
            x2.grad = None
            cd.chamfer_dist(x1, x2).backward()

        ms = _time_calls(fwd_bwd, steps, warmup, dev)
        ms_f = _time_calls(lambda: cd.ChamferFunction.apply(x1.detach(), x2.detach()), steps, warmup, dev)
        e = {"pairs": nb, "ms_fwd_bwd": round(ms, 4), "pairs_per_s": round(nb / (ms * 1e-3), 1), "ms_fwd": round(ms_f, 4),
             # all-pairs work (6 lane-ops per pair) over the time taken: above 1 where the grid search
             # skips most pairs
             "all_pairs_equiv_fp32_frac_fwd": round(6.0 * 2 * nb * N * N / (ms_f * 1e-3) / lanes, 4)}
        if ref_mod is not None:
            xd1, xd2 = x1.detach(), x2.detach()
            g1 = torch.ones(nb, N, device=dev) / (nb * N)

            def ref_fwd_bwd():
                d1, d2, i1, i2 = ref_mod.chamfer_dist(xd1, xd2)
                ref_mod.chamfer_dist_grad(xd1, xd2, i1, i2, g1, g1)

            ms_r = _time_calls(ref_fwd_bwd, max(3, steps // 2), 1, dev)
            e["reference_cuda"] = {"ms_fwd_bwd": round(ms_r, 3), "pairs_per_s": round(nb / (ms_r * 1e-3), 1),
                                   "speedup": round(ms_r / ms, 2)}
        if cpu:
            from oracle import oracle as orc

            sample = min(nb, 32 if N > 4096 else 64)
            a, b = c1[:sample].contiguous(), c2[:sample].contiguous()
            t0 = time.perf_counter()
            d1, d2, i1, i2 = orc.chamfer(a, b)
            orc.chamfer_grad(a, b, i1, i2, torch.ones(sample, N) / (nb * N), torch.ones(sample, N) / (nb * N))
            dt = time.perf_counter() - t0
            e["cpu_baseline"] = {"value": round(sample / dt, 3), "unit": "pairs/s", "cores": 1, "kind": "port",
                                 "sample": "%d of the %d pairs, forward + backward, one pass, %.1f s" % (sample, nb, dt)}
        out["B%d_N%d" % (B, N)] = e
    out["value"] = out["B%d_N%d" % shapes[0]]["pairs_per_s"]
    return out


def run_workload(args, rank=0, world=1, local_rank=0):
    """Secondary workloads, one JSON line each (rank 0):
    chamfer     B=32 pairs x N=M=16384 (and B=64 x 2048), forward + backward
    partial     64 packed scenes of 20k-200k points: partial_dense ball query and kNN k=16
    fps_large   B=8 clouds x N=2^20: FPS to --npoint (default 65536) + dense ball query
    Under torchrun (--gpus N) chamfer and fps_large split their pairs / clouds over the ranks
    (sharding.shard_range; strong scaling: the batch stays the same): the chamfer loss goes
    through the NCCL all-reduce of sharding.chamfer_dist_sharded's reduction, the per-rank
    outputs are assembled on every rank by one all_gather_into_tensor, and the time is the
    maximum over ranks between barriers."""
    import torch.distributed as dist

    import torch_points_kernels_b200 as tpk
    from torch_points_kernels_b200 import chamfer_dist as cd
    from torch_points_kernels_b200 import sharding
    from torch_points_kernels_b200 import synthetic as data

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    sm_mhz = 1965.0
    lanes = 148 * 128 * sm_mhz * 1e6
    out = {"workload": args.workload, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "data": "synthetic",
           "scaling": "strong", "higher_is_better": True}

    def timed(fn, steps, warmup):
        """ms per call: barrier + synchronize on both sides, CUDA events, maximum over ranks."""
        for _ in range(warmup):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    if args.workload == "chamfer" and world == 1:
        ref_mod, _ = load_reference_cuda()
        out.update(chamfer_numbers(dev, ref_mod, args.steps, args.warmup, cpu=not args.no_cpu_baseline))
    elif args.workload == "chamfer":
        for B, N in ((32, 16384), (64, 2048)):
            c1, c2 = data.chamfer_pair(B, N, seed=4000)
            lo, hi = sharding.shard_range(B, rank, world)
            x1, x2 = c1[lo:hi].to(dev).requires_grad_(True), c2[lo:hi].to(dev).requires_grad_(True)
            box = {}

            def step():
                x1.grad = None
                x2.grad = None
                d1, d2 = cd.ChamferFunction.apply(x1, x2)
                loss = sharding.reduce_chamfer_loss(d1.sum(), d1.numel(), d2.sum(), d2.numel())  # NCCL all-reduce
                loss.backward()
                box["loss"] = loss.detach()
                box["all"] = sharding.gather_outputs(torch.stack([d1.detach(), d2.detach()], 1), n_items=B)  # final gather

            ms = timed(step, args.steps, args.warmup)
            # every rank holds the whole batch's loss and distances; rank 0 checks them against one device
            e = {"pairs": B, "pairs_per_rank": hi - lo, "ms_fwd_bwd": round(ms, 4), "pairs_per_s": round(B / (ms * 1e-3), 1)}
            if rank == 0:
                y1, y2 = c1.to(dev), c2.to(dev)
                r1, r2 = cd.ChamferFunction.apply(y1, y2)
                want = float(r1.mean() + r2.mean())
                e["loss_rel_diff_vs_one_device"] = float("%.3g" % (abs(float(box["loss"]) - want) / want))
                e["gathered_equal_one_device"] = bool(torch.equal(box["all"][:, 0], r1) and torch.equal(box["all"][:, 1], r2))
            out["B%d_N%d" % (B, N)] = e
        out["metric"], out["unit"] = "chamfer_pairs_per_s", "pairs/s"
        out["value"] = out["B32_N16384"]["pairs_per_s"]
        out["collectives"] = "all_reduce(SUM) of 4 doubles per step (loss), all_gather_into_tensor of (pairs, 2, N) f32 (outputs)"
    elif args.workload == "partial":
        x, y, bx, by = data.packed_planes(seed=3000)
        # a contiguous block of scenes per rank, balanced by support points x queries per scene;
        # neighbour indices are made global again (+ first support point of the block) and the
        # per-rank results assembled on every rank (lists of different lengths: gather_ragged)
        s0, s1, px0, px1, py0, py1 = sharding.packed_block(bx, by, rank, world)
        xd, yd = x[px0:px1].to(dev), y[py0:py1].to(dev)
        bxd, byd = (bx[px0:px1] - s0).to(dev), (by[py0:py1] - s0).to(dev)
        box = {}

        def bq_step():
            nbr, d2 = tpk.ball_query(0.05, 64, xd, yd, mode="partial_dense", batch_x=bxd, batch_y=byd)
            box["nbr"] = sharding.gather_ragged(torch.where(nbr >= 0, nbr + px0, nbr)) if world > 1 else nbr

        def knn_step():
            idx, d2 = tpk.knn(xd, yd, 16, batch_support=bxd, batch_pos=byd)
            box["knn"] = sharding.gather_ragged(idx + px0) if world > 1 else idx

        ms_bq = timed(bq_step, args.steps, args.warmup)
        ms_knn = timed(knn_step, args.steps, args.warmup)
        nx = torch.bincount(bx).double()
        ny = torch.bincount(by, minlength=nx.numel()).double()
        pairs = float((nx * ny).sum())
        out.update({"metric": "partial_dense_ball_query_queries_per_s", "unit": "queries/s",
                    "value": round(y.shape[0] / (ms_bq * 1e-3), 1), "points": x.shape[0], "queries": y.shape[0],
                    "scenes_of_rank0": s1 - s0, "ball_query_ms": round(ms_bq, 3), "knn_k16_ms": round(ms_knn, 3),
                    "knn_queries_per_s": round(y.shape[0] / (ms_knn * 1e-3), 1), "brute_force_pairs": pairs,
                    "knn_brute_force_equiv_fp32_frac": round(6.0 * pairs / (ms_knn * 1e-3) / lanes / world, 4)})
        if world > 1:
            out["collectives"] = ("all_gather_into_tensor of the neighbour lists (queries, 64) and (queries, 16) int64, "
                                  "padded to the longest block, inside the timed calls")
            out["gathered_rows"] = [int(box["nbr"].shape[0]), int(box["knn"].shape[0])]
    elif args.workload == "fps_large":
        B, N = args.clouds or 8, 1 << 20
        m = args.npoint or 65536
        lo, hi = sharding.shard_range(B, rank, world)
        xd = data.gaussian_mixture(B, N, seed=5000)[lo:hi].to(dev)
        box = {}

        def fps_step():
            idx, centres = tpk.furthest_point_sample(xd, m, return_xyz=True)
            box["idx"], box["centres"] = idx, centres
            box["all_idx"] = sharding.gather_outputs(idx, n_items=B)  # final gather

        def bq_step():
            nbr, _ = tpk.ball_query(0.02, 32, xd, box["centres"], mode="dense")
            box["all_nbr"] = sharding.gather_outputs(nbr, n_items=B)

        if hi > lo:
            ms_fps = timed(fps_step, args.steps, 0 if world == 1 else 1)
            ms_bq = timed(bq_step, args.steps, 1)
        out.update({"metric": "large_cloud_fps_clouds_per_s", "unit": "clouds/s",
                    "value": round(B / (ms_fps * 1e-3), 4), "clouds": B, "clouds_per_rank": hi - lo, "points_per_cloud": N,
                    "npoint": m, "fps_ms": round(ms_fps, 2), "fps_us_per_round": round(ms_fps * 1e3 / (m - 1), 2),
                    "ball_query_ms": round(ms_bq, 3), "ball_query_centres_per_s": round(B * m / (ms_bq * 1e-3), 1),
                    "collectives": "all_gather_into_tensor of the sampled indices (B, npoint) int32 and of the "
                                   "neighbour lists (B, npoint, 32) int64, inside the timed calls"})
    if rank == 0:
        print(json.dumps(out), flush=True)


def run_reference_cuda(args):
    """Informational arm: the reference's own CUDA extension (compiled for sm_100a from its
    sources into oracle/_ref/points_cuda.so) on the same inputs, one GPU, its own launch
    shapes and the legacy stream choices it makes.  grouping = torch.gather on the expanded
    index, as in torchpoints.py:143-146."""
    sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
    try:
        import points_cuda as ref
    except Exception as e:
        print(json.dumps({"impl": "reference_cuda", "unavailable": "points_cuda.so does not load: %s" % e}))
        return
    from torch_points_kernels_b200 import synthetic as data

    dev = torch.device("cuda", 0)
    out = {"impl": "reference_cuda", "workload": args.workload, "steps": args.steps, "warmup": args.warmup}
    if args.workload == "sa_fp_pipeline":
        B, N = B_CLOUDS, N_POINTS
        xyz_h, sa_h, fp_h = make_inputs(B, N, 2000)
        dev_in = [xyz_h.to(dev)] + [t.to(dev) for t in sa_h] + [t.to(dev) for t in fp_h]
        pipe = Pipeline(dev, B, N, 2000)
        res, _ = time_reference_cuda(ref, dev, dev_in, lambda ts: (ts[0], list(ts[1:5]), list(ts[5:9])), pipe,
                                     args.steps, args.in_flight)
        out.update({"metric": METRIC, "unit": "clouds/s", "value": res["clouds_per_s_isolated"]})
        out.update(res)
    elif args.workload == "chamfer":
        for B, N in ((32, 16384), (64, 2048)):
            c1, c2 = data.chamfer_pair(B, N, seed=4000)
            x1, x2 = c1.to(dev), c2.to(dev)
            g1, g2 = torch.ones(B, N, device=dev) / (B * N), torch.ones(B, N, device=dev) / (B * N)

            def fwd_bwd():
                d1, d2, i1, i2 = ref.chamfer_dist(x1, x2)
                ref.chamfer_dist_grad(x1, x2, i1, i2, g1, g2)

            ms = _time_calls(fwd_bwd, args.steps, args.warmup, dev)
            out["B%d_N%d" % (B, N)] = {"ms_fwd_bwd": round(ms, 3), "pairs_per_s": round(B / (ms * 1e-3), 1)}
    elif args.workload == "partial":
        x, y, bx, by = data.packed_planes(seed=3000)
        xd, yd, bxd, byd = x.to(dev), y.to(dev), bx.to(dev), by.to(dev)
        ms = _time_calls(lambda: ref.ball_query_partial_dense(xd, yd, bxd, byd, 0.05, 64), args.steps, args.warmup, dev)
        out.update({"ball_query_ms": round(ms, 2), "queries_per_s": round(y.shape[0] / (ms * 1e-3), 1)})
    elif args.workload == "fps_large":
        B, N = args.clouds or 8, 1 << 20
        m = args.npoint or 65536
        xd = data.gaussian_mixture(B, N, seed=5000).to(dev)
        ms = _time_calls(lambda: ref.furthest_point_sampling(xd, m), args.steps, 0, dev)
        out.update({"fps_ms": round(ms, 2), "fps_us_per_round": round(ms * 1e3 / (m - 1), 2), "npoint": m})
    print(json.dumps(out), flush=True)


def run_only(args):
    """One op of the stack at its pipeline shape (optionally fewer clouds / samples), for
    profiler captures of a single kernel:  --only fps_l1|ball_query_l2|grouping_bwd_l1|...
    Prints the mean time per launch."""
    import torch_points_kernels_b200 as tpk

    dev = torch.device("cuda", 0)
    B = args.clouds or B_CLOUDS
    name, lvl = args.only.rsplit("_l", 1)
    l = int(lvl) - 1
    xyz_h, sa_h, fp_h = make_inputs(B, N_POINTS, 2000)
    pts = [xyz_h.to(dev)]
    for i in range(l + 1):  # geometry of the levels below (untimed setup)
        m = LEVELS["npoint"][i] if not (i == l and args.npoint) else args.npoint
        idx = tpk.furthest_point_sample(pts[i], m)
        pts.append(torch.gather(pts[i], 1, idx.long().unsqueeze(-1).expand(-1, -1, 3)).contiguous())
    m = pts[l + 1].shape[1]
    fps_idx_l = idx
    r, ns, c = LEVELS["radius"][l], LEVELS["nsample"], LEVELS["channels"][l]
    g = torch.Generator(device=dev).manual_seed(3)
    feat = sa_h[l].to(dev)
    ffeat = torch.randn(B, c, m, device=dev, generator=g)
    nbr, _ = tpk.ball_query(r, ns, pts[l], pts[l + 1], mode="dense")
    dist, idx3 = tpk.three_nn(pts[l], pts[l + 1])
    w = 1.0 / (dist + 1e-8)
    w = (w / w.sum(dim=2, keepdim=True)).contiguous()
    g_grouped = torch.randn(B, c, m, ns, device=dev, generator=g)
    g_up = torch.randn(B, c, pts[l].shape[1], device=dev, generator=g)
    ops = {
        "fps": lambda: tpk.furthest_point_sample(pts[l], m),
        "ball_query": lambda: tpk.ball_query(r, ns, pts[l], pts[l + 1], mode="dense"),
        "three_nn": lambda: tpk.three_nn(pts[l], pts[l + 1]),
        "grouping_fwd": lambda: tpk.grouping_operation(feat, nbr),
        "grouping_bwd": lambda: tpk.torchpoints.grouping_backward(g_grouped, nbr, feat.shape[2]),
        "interp_fwd": lambda: tpk.three_interpolate(ffeat, idx3, w),
        "sa_group": lambda: tpk.sa_group(pts[l], feat, fps_idx_l, r, ns),
        "interp_bwd": lambda: tpk.torchpoints.three_interpolate_backward(g_up, idx3, w, m),
    }
    fn = ops[name]
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize(dev)
    run = fn
    if args.graph:
        # device time of the op alone: its launches replayed from a CUDA graph, no host work between them
        side = torch.cuda.Stream(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
            fn()
        run = graph.replay
        run()
        torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize(dev)
    print(json.dumps({"only": args.only, "clouds": B, "npoint": m, "steps": args.steps, "graph": bool(args.graph),
                      "ms_per_call": round(e0.elapsed_time(e1) / args.steps, 4)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, help="run one op of the stack, e.g. fps_l1, grouping_bwd_l1")
    ap.add_argument("--clouds", type=int, default=0, help="with --only: clouds per batch (default 16)")
    ap.add_argument("--npoint", type=int, default=0, help="with --only: samples of that level's FPS")
    ap.add_argument("--graph", action="store_true", help="with --only: time the op replayed from a CUDA graph")
    ap.add_argument("--workload", default="sa_fp_pipeline", choices=["sa_fp_pipeline", "chamfer", "partial", "fps_large"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference_cuda"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-cuda", action="store_true",
                    help="skip timing the reference's CUDA build and checking the step's results against it")
    ap.add_argument("--no-chamfer", action="store_true", help="skip the chamfer pairs/s leg of the default run")
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="the timed region of --steps steps is repeated until the repetitions cover this long")
    ap.add_argument("--in-flight", type=int, default=8, help="CUDA graphs (steps) replayed in rotation, each on its own stream")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel from Python instead of replaying CUDA graphs")
    args = ap.parse_args()
    if args.impl == "b200" and not args.only and args.workload == "sa_fp_pipeline":
        args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.impl == "reference_cuda":
        run_reference_cuda(args)
        return
    if args.only:
        run_only(args)
        return
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload != "sa_fp_pipeline":
            run_workload(args, rank, world, local_rank)
        else:
            run_b200(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
