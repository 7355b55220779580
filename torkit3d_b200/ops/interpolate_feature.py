"""Weighted three-neighbour feature interpolation (torkit3d/ops/interpolate_feature.py:27-40)."""
import torch

from .. import _C
from ._functions import InterpolateFeature

__all__ = ["interpolate_feature", "three_nn_weight", "feature_rows", "InterpolateFeature"]


def interpolate_feature(feature: torch.Tensor, index: torch.Tensor, weight: torch.Tensor, rows: torch.Tensor = None):
    """out[b, c, m] = sum_i feature[b, c, index[b, m, i]] * weight[b, m, i]  (i over 3 neighbours).

    Args:
        feature: [B, C, N1] key-point features.
        index: [B, N2, 3] int64.
        weight: [B, N2, 3].
        rows: optional ``feature_rows(feature)`` (an addition to the reference's signature): the
            forward pass then skips its per-call transposition of the features.

    Returns:
        [B, C, N2]; differentiable w.r.t. ``feature``.
    """
    if rows is None:
        return InterpolateFeature.apply(feature, index, weight)
    return InterpolateFeature.apply(feature, index, weight, rows)


def feature_rows(feature: torch.Tensor) -> torch.Tensor:
    """[B, C, N] float32 features as rows [B, N, C], the layout the large gathers read.

    ``interpolate_feature`` and ``group_points`` build this copy on every call when their output
    is large; a caller that gathers from the same features several times (query slabs of one scene
    spread over calls or GPUs, several groupings of one cloud) builds it once and passes it as
    ``rows=``.  Not differentiable: gradients flow through the ``feature`` argument of the gather.
    """
    return _C.feature_rows(feature.detach().contiguous())


def three_nn_weight(distance: torch.Tensor) -> torch.Tensor:
    """Normalised inverse squared-distance weights, 1/max(d, 1e-10) / sum, over the last axis.

    One kernel for the four element-wise PyTorch ops of ``FeatureInterpolator.forward``
    (torkit3d/layers/pointnet2.py:128-130).  ``distance`` is what ``knn_points`` returns (squared).
    """
    return _C.three_nn_weight_cuda(distance.contiguous())
