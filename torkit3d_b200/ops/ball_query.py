"""Ball query (public signature of torkit3d/ops/ball_query.py:17-38)."""
import torch

from ._functions import BallQueryFunction

__all__ = ["ball_query", "BallQueryFunction"]


def ball_query(query: torch.Tensor, key: torch.Tensor, radius, max_neighbors, transpose=True, *,
               index_dtype=torch.int64):
    """First ``max_neighbors`` key indices (ascending) strictly inside ``radius`` of each query.

    Args:
        query: [B, 3, N1] ([B, N1, 3] when ``transpose`` is False).
        key: [B, 3, N2] ([B, N2, 3] when ``transpose`` is False).
        radius: ball radius (squared in the tensors' dtype after conversion to a C float).
        max_neighbors: K; rows with fewer hits repeat their first hit, rows with none are -1.
        transpose: inputs are channel-first (the default, as in the reference).
        index_dtype: ``torch.int64`` (the reference's type) or, as an opt-in, ``torch.int32``.

    Returns:
        index [B, N1, K].
    """
    # channel-first clouds are read in place (the reference copies them: torkit3d/ops/ball_query.py:32-36)
    return BallQueryFunction.apply(query, key, radius, max_neighbors, bool(transpose), index_dtype)
