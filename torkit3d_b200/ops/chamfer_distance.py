"""Chamfer distance (public signatures of torkit3d/ops/chamfer_distance.py:32-71)."""
import torch

from .. import _C
from ._functions import ChamferDistanceFunction, pick_layout

__all__ = ["chamfer_distance", "nn_distance", "safe_sqrt", "ChamferDistanceFunction"]


def safe_sqrt(x, eps=1e-12):
    """sqrt(max(x, eps)): keeps the gradient finite at zero distance."""
    return torch.clamp(x, eps).sqrt()


def _batched(xyz):
    return xyz.unsqueeze(0) if xyz.dim() == 2 else xyz


def chamfer_distance(xyz1, xyz2, transpose=False, sqrt=False, eps=1e-12):
    """Squared (or, with ``sqrt``, Euclidean) distance from every point to the other cloud.

    Args:
        xyz1: [B, N1, 3] (or [N1, 3]); [B, 3, N1] when ``transpose`` is set.
        xyz2: [B, N2, 3] (or [N2, 3]); [B, 3, N2] when ``transpose`` is set.
        transpose: inputs are channel-first and must be transposed first.
        sqrt: return sqrt(clamp(d, eps)) instead of the squared distance.
        eps: clamp for ``sqrt``.

    Returns:
        dist1 [B, N1], dist2 [B, N2].  Differentiable w.r.t. both clouds.
    """
    xyz1, xyz2 = _batched(xyz1), _batched(xyz2)
    # channel-first clouds are read, and their gradients written, in place (the reference transposes
    # and copies both: torkit3d/ops/chamfer_distance.py:49-52)
    dist1, dist2 = ChamferDistanceFunction.apply(xyz1, xyz2, bool(transpose))
    if sqrt:
        dist1, dist2 = safe_sqrt(dist1, eps), safe_sqrt(dist2, eps)
    return dist1, dist2


def nn_distance(xyz1, xyz2, transpose=False):
    """Inference-time variant without autograd: returns [dist1, idx1, dist2, idx2]."""
    xyz1, xyz2 = _batched(xyz1), _batched(xyz2)
    cf, xyz1, xyz2 = pick_layout(transpose, xyz1, xyz2)
    return _C.chamfer_distance_forward_cuda(xyz1, xyz2, channel_first=cf)
