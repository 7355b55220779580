"""The six ``torch.autograd.Function`` classes of the operator layer.

Class names, ``forward`` argument lists and the tensors kept for backward are those of the
reference (``torkit3d/ops/*.py``), so code that reaches for ``ChamferDistanceFunction.apply`` or
relies on what is saved for ``torch.utils.checkpoint`` keeps working.  All of them call the
``_C``-compatible shim, which in turn calls the C ABI of libtk3d_b200.so; none has a CPU path.
"""
import torch

from .. import _C


def _no_grads(n):
    return (None,) * n


class ChamferDistanceFunction(torch.autograd.Function):
    """(xyz1, xyz2) -> (dist1, dist2); saves (xyz1, xyz2, idx1, idx2).
    Reference: torkit3d/ops/chamfer_distance.py:10-29."""

    @staticmethod
    def forward(ctx, xyz1, xyz2):
        a, b = xyz1.contiguous(), xyz2.contiguous()
        if not (a.is_cuda and b.is_cuda):
            raise AssertionError("Only support cuda currently.")
        dist1, idx1, dist2, idx2 = _C.chamfer_distance_forward_cuda(a, b)
        ctx.save_for_backward(a, b, idx1, idx2)
        return dist1, dist2

    @staticmethod
    def backward(ctx, grad_dist1, grad_dist2):
        a, b, idx1, idx2 = ctx.saved_tensors
        g1, g2 = grad_dist1.contiguous(), grad_dist2.contiguous()
        if not (g1.is_cuda and g2.is_cuda):
            raise AssertionError("Only support cuda currently.")
        grad_a, grad_b = _C.chamfer_distance_backward_cuda(g1, g2, a, b, idx1, idx2)
        return grad_a, grad_b


class KNNDistanceFunction(torch.autograd.Function):
    """(query, key, k, version) -> (distance, index); no gradients.
    Reference: torkit3d/ops/knn_points.py:6-13."""

    @staticmethod
    def forward(ctx, query_xyz, key_xyz, k, version):
        distance, index = _C.knn_distance_cuda(query_xyz, key_xyz, k, version)
        return distance, index

    @staticmethod
    def backward(ctx, *grad_outputs):
        return _no_grads(4)


class SampleFarthestPointsFunction(torch.autograd.Function):
    """(points, num_samples) -> index; no gradients.
    Reference: torkit3d/ops/sample_farthest_points.py:6-14."""

    @staticmethod
    def forward(ctx, points, num_samples):
        index = _C.sample_farthest_points_cuda(points, num_samples)
        return index

    @staticmethod
    def backward(ctx, *grad_outputs):
        return _no_grads(2)


class BallQueryFunction(torch.autograd.Function):
    """(query, key, radius, max_neighbors) -> index; no gradients.
    Reference: torkit3d/ops/ball_query.py:6-14."""

    @staticmethod
    def forward(ctx, query, key, radius, max_neighbors):
        index = _C.ball_query_cuda(query, key, radius, max_neighbors)
        return index

    @staticmethod
    def backward(ctx, *grad_outputs):
        return _no_grads(4)


class GroupPointsFunction(torch.autograd.Function):
    """(points [B,C,N1], index [B,N2,K]) -> [B,C,N2,K]; saves index and N1.
    Reference: torkit3d/ops/group_points.py:6-19."""

    @staticmethod
    def forward(ctx, points, index):
        ctx.save_for_backward(index)
        ctx.num_points = points.size(2)
        return _C.group_points_forward_cuda(points.contiguous(), index.contiguous())

    @staticmethod
    def backward(ctx, *grad_output):
        (index,) = ctx.saved_tensors
        grad_points = _C.group_points_backward_cuda(grad_output[0].contiguous(), index.contiguous(), ctx.num_points)
        return grad_points, None


class InterpolateFeature(torch.autograd.Function):
    """(feature [B,C,N1], index [B,N2,3], weight [B,N2,3]) -> [B,C,N2]; gradient for feature only.
    Reference: torkit3d/ops/interpolate_feature.py:6-24."""

    @staticmethod
    def forward(ctx, feature, index, weight):
        ctx.save_for_backward(index, weight)
        ctx.n1 = feature.size(2)
        return _C.interpolate_forward_cuda(feature.contiguous(), index.contiguous(), weight.contiguous())

    @staticmethod
    def backward(ctx, *grad_out):
        index, weight = ctx.saved_tensors
        grad_feature = _C.interpolate_backward_cuda(grad_out[0].contiguous(), index.contiguous(),
                                                    weight.contiguous(), ctx.n1)
        return grad_feature, None, None
