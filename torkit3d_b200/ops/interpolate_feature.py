"""Weighted three-neighbour feature interpolation (torkit3d/ops/interpolate_feature.py:27-40)."""
import torch

from .. import _C
from ._functions import InterpolateFeature

__all__ = ["interpolate_feature", "three_nn_weight", "InterpolateFeature"]


def interpolate_feature(feature: torch.Tensor, index: torch.Tensor, weight: torch.Tensor):
    """out[b, c, m] = sum_i feature[b, c, index[b, m, i]] * weight[b, m, i]  (i over 3 neighbours).

    Args:
        feature: [B, C, N1] key-point features.
        index: [B, N2, 3] int64.
        weight: [B, N2, 3].

    Returns:
        [B, C, N2]; differentiable w.r.t. ``feature``.
    """
    return InterpolateFeature.apply(feature, index, weight)


def three_nn_weight(distance: torch.Tensor) -> torch.Tensor:
    """Normalised inverse squared-distance weights, 1/max(d, 1e-10) / sum, over the last axis.

    One kernel for the four element-wise PyTorch ops of ``FeatureInterpolator.forward``
    (torkit3d/layers/pointnet2.py:128-130).  ``distance`` is what ``knn_points`` returns (squared).
    """
    return _C.three_nn_weight_cuda(distance.contiguous())
