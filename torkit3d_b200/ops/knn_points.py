"""k nearest neighbours with distances (public signature of torkit3d/ops/knn_points.py:16-51)."""
import torch

from ._functions import KNNDistanceFunction

__all__ = ["knn_points", "KNNDistanceFunction"]


def knn_points(query: torch.Tensor, key: torch.Tensor, k: int, sorted: bool = False, sqrt_distance: bool = False,
               transpose: bool = False, version: int = 1, *, index_dtype=torch.int64):
    """For every query point the k nearest key points.

    Args:
        query: [B, N1, 3] ([B, 3, N1] when ``transpose``).
        key: [B, N2, 3] ([B, 3, N2] when ``transpose``); N2 >= k.
        k: number of neighbours.
        sorted: ask for rows in ascending distance order.  The kernels here always emit rows sorted
            by (distance, index), so this costs nothing; the flag is kept for compatibility.
        sqrt_distance: return Euclidean instead of squared distances.
        transpose: inputs are channel-first.
        version: kernel selector of the reference (0 or 1); both map to the same kernels here.
        index_dtype: ``torch.int64`` (the reference's type) or, as an opt-in, ``torch.int32``.

    Returns:
        (distance [B, N1, k], index [B, N1, k]) -- in this order, as the reference returns them.
    """
    # channel-first clouds are read in place (the reference copies them: torkit3d/ops/knn_points.py:40-44)
    distance, index = KNNDistanceFunction.apply(query, key, k, version, bool(transpose), index_dtype)
    if sqrt_distance:
        distance = distance.sqrt()
    return distance, index
