"""Operator layer: same public names as ``torkit3d.ops``."""
from .ball_query import ball_query
from .chamfer_distance import chamfer_distance, nn_distance
from .edge_conv import get_edge_feature
from .group_points import group_points
from .interpolate_feature import feature_rows, interpolate_feature, three_nn_weight
from .knn_points import knn_points
from .native import knn
from .sample_farthest_points import sample_farthest_points

__all__ = ["ball_query", "chamfer_distance", "nn_distance", "group_points", "interpolate_feature",
           "three_nn_weight", "feature_rows", "knn_points", "knn", "sample_farthest_points", "get_edge_feature"]
