"""Instance IoU (reference: torch_points_kernels/metrics.py, kernel cuda/src/metrics_gpu.cu)."""
from typing import List, Optional

import torch

from . import _lib


def instance_iou(
    instance_idx: List[torch.Tensor],
    gt_instances: torch.Tensor,
    batch: Optional[torch.Tensor] = None,
):
    """Computes the IoU between each proposed instance in instance_idx and ground truth instances. Returns a
    tensor of shape [instance_idx.shape[0], num_instances] that contains the iou between the proposed instances and all gt instances
    Instance label 0 is reserved for non instance points

    Parameters
    ----------
    instance_idx : List[torch.Tensor]
        List of instances. Each tensor in this list is a proposed and contains the index of the points
        that belong to that particular instance
    gt_instances : torch.Tensor
        Ground truth instances, contains the index of the instance for each point

    Returns
    -------
    ious: torch.Tensor[nb_proposals, nb_groundtruth]
    """
    _lib.check_cuda(gt_instances, "gt_instances")
    dev = gt_instances.device
    gt_instances = gt_instances.long().contiguous()
    if batch is None:
        batch = torch.zeros_like(gt_instances)
    batch = batch.long().to(dev).contiguous()

    # Number of gt instances per sample (the largest label of the sample) and their sizes, on the
    # device: the reference loops over samples and instances in Python (metrics.py:63-74)
    batch_size = int(batch[-1].item()) + 1
    num_gt_instances = torch.zeros(batch_size, dtype=torch.long, device=dev).scatter_reduce_(
        0, batch, gt_instances.clamp(min=0), reduce="amax", include_self=True)
    offset_num_gt = torch.cat([torch.zeros(1, dtype=torch.long, device=dev), num_gt_instances.cumsum(0)])
    total_gt = int(offset_num_gt[-1].item())
    max_gt = int(num_gt_instances.max().item()) if batch_size else 0
    is_inst = gt_instances >= 1
    key = offset_num_gt[batch[is_inst]] + gt_instances[is_inst] - 1
    gt_instance_sizes = torch.bincount(key, minlength=max(total_gt, 1))[:total_gt].contiguous()

    offsets = [0]
    for instance in instance_idx:
        offsets.append(offsets[-1] + instance.shape[0])
    proposals_offset = torch.tensor(offsets, dtype=torch.long, device=dev)
    proposals_idx = torch.cat([i.to(dev).long() for i in instance_idx]).contiguous() if instance_idx else \
        torch.zeros(0, dtype=torch.long, device=dev)
    out = torch.empty((len(instance_idx), total_gt), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("tpk_instance_iou", len(instance_idx), total_gt, max_gt, gt_instances.shape[0],
                  _lib.ptr(num_gt_instances), _lib.ptr(proposals_idx), _lib.ptr(proposals_offset),
                  _lib.ptr(gt_instances), _lib.ptr(offset_num_gt), _lib.ptr(batch), _lib.ptr(gt_instance_sizes),
                  _lib.ptr(out), _lib.stream_of(gt_instances))
    return out
