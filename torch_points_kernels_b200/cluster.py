"""Region growing on the GPU (reference: torch_points_kernels/cluster.py, a numba traversal on
the CPU there).  The neighbour search is the packed ball query; the clusters come from label
propagation on the device (tpk_grow_labels_step) instead of a sequential traversal."""
import ctypes
from typing import List

import torch

from . import _lib
from .torchpoints import ball_query_partial_dense


def cluster_labels(neighbours):
    """neighbours: (N, nsample) int64 CUDA tensor of neighbour lists (-1 ends a list).  Returns
    (N,) int32 labels: labels[v] = smallest index that reaches v along the lists = seed of the
    cluster the reference's traversal (cluster.py:8-37) assigns v to."""
    _lib.check_cuda(neighbours, "neighbours")
    if neighbours.dtype != torch.int64:
        raise RuntimeError("neighbours must be an int64 tensor")
    neighbours = neighbours.contiguous()
    n, nsample = neighbours.shape
    labels = torch.arange(n, dtype=torch.int32, device=neighbours.device)
    changed = torch.zeros(1, dtype=torch.int32, device=neighbours.device)
    with torch.cuda.device(neighbours.device):
        # chains shorten geometrically; a handful of launches per host check keeps the number of
        # device-to-host reads small
        for _ in range(max(1, n)):
            changed.zero_()
            _lib.call("tpk_grow_labels_step", n, nsample, _lib.ptr(neighbours), _lib.ptr(labels), _lib.ptr(changed),
                      8, _lib.stream_of(neighbours))
            if int(changed.item()) == 0:
                break
    return labels


def grow_proximity(pos, batch, nsample=16, radius=0.02, min_cluster_size=32):
    """Grow based on proximity only.  Returns the clusters as lists of point indices, ordered by
    their smallest member; the members of a cluster are listed in ascending order (the reference
    lists them in the order its traversal met them: the sets are the same)."""
    assert pos.shape[0] == batch.shape[0]
    pos = pos.float().contiguous()
    neighbours = ball_query_partial_dense(radius, nsample, pos, pos, batch, batch)[0]
    labels = cluster_labels(neighbours)
    order = torch.sort(labels.long(), stable=True).indices  # members ascending inside a label
    seeds, counts = torch.unique_consecutive(labels[order], return_counts=True)
    clusters = []
    start = 0
    order_h, counts_h = order.cpu(), counts.cpu().tolist()
    for c in counts_h:
        if c >= min_cluster_size:
            clusters.append(order_h[start:start + c].tolist())
        start += c
    return clusters


def region_grow(
    pos, labels, batch, ignore_labels=[], nsample=16, radius=0.02, min_cluster_size=32
) -> List[torch.Tensor]:
    """Region growing clustering algorithm proposed in
    PointGroup: Dual-Set Point Grouping for 3D Instance Segmentation
    https://arxiv.org/pdf/2004.01658.pdf
    for instance segmentation

    Parameters
    ----------
    pos: torch.Tensor [N, 3]
        Location of the points
    labels: torch.Tensor [N,]
        labels of each point
    ignore_labels:
        Labels that should be ignored, no region growing will be performed on those
    nsample:
        maximum number of neighbours to consider
    radius:
        radius for the neighbour search
    min_cluster_size:
        Number of points above which a cluster is considered valid
    """
    assert labels.dim() == 1
    assert pos.dim() == 2
    assert pos.shape[0] == labels.shape[0]

    unique_labels = torch.unique(labels)
    clusters = []
    ind = torch.arange(0, pos.shape[0], device=pos.device)
    for l in unique_labels:
        if l in ignore_labels:
            continue

        # Build clusters for a given label (ignore other points)
        label_mask = labels == l
        local_ind = ind[label_mask]

        # Remap batch to a continuous sequence (batch is sorted, so is the remapped vector)
        label_batch = batch[label_mask]
        remaped_batch = torch.unique(label_batch, return_inverse=True)[1]

        # Cluster
        label_clusters = grow_proximity(
            pos[label_mask, :],
            remaped_batch,
            nsample=nsample,
            radius=radius,
            min_cluster_size=min_cluster_size,
        )

        # Remap indices to original coordinates
        for cluster in label_clusters:
            cluster = torch.tensor(cluster, device=pos.device)
            clusters.append(local_ind[cluster])

    return clusters
