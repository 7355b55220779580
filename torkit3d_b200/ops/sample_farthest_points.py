"""Farthest point sampling (public signature of torkit3d/ops/sample_farthest_points.py:17-31)."""
import torch

from ._functions import SampleFarthestPointsFunction

__all__ = ["sample_farthest_points", "SampleFarthestPointsFunction"]


def sample_farthest_points(points: torch.Tensor, num_samples, transpose=False):
    """Indices [B, num_samples] of iteratively farthest points, starting from point 0.

    Args:
        points: [B, N, 3] ([B, 3, N] when ``transpose``).
        num_samples: number of points to pick, 1 <= num_samples <= N.
        transpose: input is channel-first.
    """
    # a channel-first cloud is read in place (the reference copies it: torkit3d/ops/sample_farthest_points.py:28-30)
    return SampleFarthestPointsFunction.apply(points, num_samples, bool(transpose))
