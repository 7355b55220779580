"""Gather point features by neighbour index (signature of torkit3d/ops/group_points.py:22-32)."""
import torch

from ._functions import GroupPointsFunction

__all__ = ["group_points", "GroupPointsFunction"]


def group_points(points: torch.Tensor, index: torch.Tensor, rows: torch.Tensor = None) -> torch.Tensor:
    """out[b, c, m, j] = points[b, c, index[b, m, j]].

    Args:
        points: [B, C, N1] features.
        index: [B, N2, K] int64 (or int32) neighbour indices in [0, N1).
        rows: optional ``feature_rows(points)`` (an addition to the reference's signature) for
            callers that group the same features several times.

    Returns:
        [B, C, N2, K]; differentiable w.r.t. ``points``.
    """
    if rows is None:
        return GroupPointsFunction.apply(points, index)
    return GroupPointsFunction.apply(points, index, rows)
