"""Pure-PyTorch KNN on arbitrary feature dimension (signature of torkit3d/ops/native.py:4-30).

This is the one operator of the layer that is not backed by the CUDA library: the reference
defines it as ``cdist`` + ``topk`` and models call it on D-dimensional features.
"""
import torch

__all__ = ["knn"]


def knn(query: torch.Tensor, key: torch.Tensor, k: int, sorted: bool = False, transpose: bool = False):
    """Returns (Euclidean distance [B, N1, k], index [B, N1, k]) of the k nearest keys."""
    if transpose:
        query, key = query.transpose(1, 2), key.transpose(1, 2)
    pairwise = torch.cdist(query, key)
    return torch.topk(pairwise, k, dim=2, largest=False, sorted=sorted)
