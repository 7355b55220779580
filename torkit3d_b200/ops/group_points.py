"""Gather point features by neighbour index (signature of torkit3d/ops/group_points.py:22-32)."""
import torch

from ._functions import GroupPointsFunction

__all__ = ["group_points", "GroupPointsFunction"]


def group_points(points: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """out[b, c, m, j] = points[b, c, index[b, m, j]].

    Args:
        points: [B, C, N1] features.
        index: [B, N2, K] int64 neighbour indices in [0, N1).

    Returns:
        [B, C, N2, K]; differentiable w.r.t. ``points``.
    """
    return GroupPointsFunction.apply(points, index)
