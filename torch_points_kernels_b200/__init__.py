"""B200 (sm_100a) drop-in for the spatial-search path of torch-points-kernels.

Exports the reference's names for that path: furthest_point_sample, ball_query
(dense and partial_dense), knn, three_nn, three_interpolate, grouping_operation;
``chamfer_dist`` is a submodule, as in the reference.  Next to the path: region growing
(``region_grow``, ``grow_proximity``), ``instance_iou`` and the GRNet ops ``gridding`` and
``cubic_feature_sampling``, under the reference's names.
"""
from .torchpoints import (  # noqa: F401
    ball_query,
    ball_query_dense,
    ball_query_partial_dense,
    furthest_point_sample,
    grouping_operation,
    sa_group,
    three_interpolate,
    three_nn,
    ThreeInterpolate,
    GroupingOperation,
)
from .knn import knn  # noqa: F401
from . import chamfer_dist  # noqa: F401
from .cluster import grow_proximity, region_grow  # noqa: F401
from .cubic_feature_sampling import cubic_feature_sampling  # noqa: F401
from . import gridding  # noqa: F401  (a submodule, like chamfer_dist)
from .metrics import instance_iou  # noqa: F401

__all__ = [
    "ball_query",
    "furthest_point_sample",
    "grouping_operation",
    "three_interpolate",
    "three_nn",
    "knn",
    "chamfer_dist",
    "region_grow",
    "grow_proximity",
    "instance_iou",
    "gridding",
    "cubic_feature_sampling",
]
