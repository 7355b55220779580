"""KNN on an arbitrary feature dimension (signature of torkit3d/ops/native.py:4-30).

The reference defines it as ``cdist`` + ``topk`` in plain PyTorch and its models call it on
D-dimensional features (DGCNN's dynamic graph).  Float32 CUDA tensors with k <= 128 are served by the
library's feature-space kernel (``tk3d_feature_knn``); everything else runs the reference's own
formulation on whatever device the tensors live on, as the reference does.
"""
import torch

from .. import _C

__all__ = ["knn"]


def knn(query: torch.Tensor, key: torch.Tensor, k: int, sorted: bool = False, transpose: bool = False):
    """Returns (Euclidean distance [B, N1, k], index [B, N1, k]) of the k nearest keys.

    query [B, N1, D], key [B, N2, D]; [B, D, N1], [B, D, N2] if ``transpose``.  The CUDA path always
    returns rows sorted by (distance, index), which satisfies both values of ``sorted``; when an
    input requires grad the k returned distances are recomputed from the selected pairs with
    PyTorch operations so that they stay differentiable, as cdist's are.
    """
    if (query.is_cuda and key.is_cuda and query.dtype == torch.float32 and key.dtype == torch.float32
            and query.dim() == 3 and key.dim() == 3 and 1 <= k <= 128):
        d2, index = _C.feature_knn_cuda(query.detach().contiguous(), key.detach().contiguous(), k,
                                        channel_first=transpose)
        if not (torch.is_grad_enabled() and (query.requires_grad or key.requires_grad)):
            return torch.sqrt(d2), index
        # Distances that take part in autograd: recomputed for the k selected pairs only.
        qf, kf = (query.transpose(1, 2), key.transpose(1, 2)) if transpose else (query, key)
        batch = torch.arange(qf.size(0), device=qf.device).view(-1, 1, 1)
        return (kf[batch, index] - qf.unsqueeze(2)).norm(dim=-1), index
    if transpose:
        query, key = query.transpose(1, 2), key.transpose(1, 2)
    pairwise = torch.cdist(query, key)
    return torch.topk(pairwise, k, dim=2, largest=False, sorted=sorted)
