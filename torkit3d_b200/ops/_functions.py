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


def pick_layout(transpose, *clouds):
    """Choose how to hand coordinate tensors to the kernels without copying them.

    ``transpose`` is the operators' flag: the tensors are [B,3,N] when set, [B,N,3] otherwise.  The
    kernels read either layout in place, so a tensor that is contiguous as given goes through
    untouched (``channel_first`` = ``transpose``); one that is a transposed view of the other
    layout (what ``.transpose(1, 2)`` of a contiguous tensor is) goes through as that underlying
    tensor with the flag flipped.  Only tensors that are dense in neither reading, or that disagree
    with the others, are copied -- the reference copies every channel-first input
    (torkit3d/ops/ball_query.py:32-36, ops/knn_points.py:40-44, ops/sample_farthest_points.py:28-30).
    Returns (channel_first, tensors...).
    """
    transpose = bool(transpose)
    if all(t.is_contiguous() for t in clouds):
        return (transpose,) + tuple(clouds)
    flipped = [t.transpose(1, 2) for t in clouds]
    if all(t.is_contiguous() for t in flipped):
        return (not transpose,) + tuple(flipped)
    return (transpose,) + tuple(t.contiguous() for t in clouds)


class ChamferDistanceFunction(torch.autograd.Function):
    """(xyz1, xyz2) -> (dist1, dist2); saves (xyz1, xyz2, idx1, idx2).
    Reference: torkit3d/ops/chamfer_distance.py:10-29."""

    @staticmethod
    def forward(ctx, xyz1, xyz2, *extra):
        # [B,N,3] clouds, or [B,3,N] when a third argument (channel_first, an addition to the
        # reference's signature) is true; either way a dense tensor, or a transposed view of one,
        # is read in place
        channel_first = bool(extra[0]) if extra else False
        cf, a, b = pick_layout(channel_first, xyz1, xyz2)
        if not (a.is_cuda and b.is_cuda):
            raise AssertionError("Only support cuda currently.")
        dist1, idx1, dist2, idx2 = _C.chamfer_distance_forward_cuda(a, b, channel_first=cf)
        ctx.save_for_backward(a, b, idx1, idx2)
        ctx.kernel_cf = cf
        ctx.flipped = cf != channel_first
        ctx.n_extra = len(extra)
        return dist1, dist2

    @staticmethod
    def backward(ctx, grad_dist1, grad_dist2):
        a, b, idx1, idx2 = ctx.saved_tensors
        g1, g2 = grad_dist1.contiguous(), grad_dist2.contiguous()
        if not (g1.is_cuda and g2.is_cuda):
            raise AssertionError("Only support cuda currently.")
        grad_a, grad_b = _C.chamfer_distance_backward_cuda(g1, g2, a, b, idx1, idx2, channel_first=ctx.kernel_cf)
        if ctx.flipped:  # the kernels saw the transposed view of the inputs
            grad_a, grad_b = grad_a.transpose(1, 2), grad_b.transpose(1, 2)
        return (grad_a, grad_b) + _no_grads(ctx.n_extra)


class KNNDistanceFunction(torch.autograd.Function):
    """(query, key, k, version) -> (distance, index); no gradients.
    Reference: torkit3d/ops/knn_points.py:6-13."""

    @staticmethod
    def forward(ctx, query_xyz, key_xyz, k, version, *extra):
        # extra (additions to the reference's signature): channel_first, index_dtype
        channel_first = bool(extra[0]) if len(extra) > 0 else False
        index_dtype = extra[1] if len(extra) > 1 else torch.int64
        cf, q, r = pick_layout(channel_first, query_xyz, key_xyz)
        distance, index = _C.knn_distance_cuda(q, r, k, version, channel_first=cf, index_dtype=index_dtype)
        ctx.mark_non_differentiable(distance, index)
        ctx.n_args = 4 + len(extra)
        return distance, index

    @staticmethod
    def backward(ctx, *grad_outputs):
        return _no_grads(ctx.n_args)


class SampleFarthestPointsFunction(torch.autograd.Function):
    """(points, num_samples) -> index; no gradients.
    Reference: torkit3d/ops/sample_farthest_points.py:6-14."""

    @staticmethod
    def forward(ctx, points, num_samples, *extra):
        # extra (an addition to the reference's signature): channel_first
        cf, p = pick_layout(bool(extra[0]) if extra else False, points)
        index = _C.sample_farthest_points_cuda(p, num_samples, channel_first=cf)
        ctx.mark_non_differentiable(index)
        ctx.n_args = 2 + len(extra)
        return index

    @staticmethod
    def backward(ctx, *grad_outputs):
        return _no_grads(ctx.n_args)


class BallQueryFunction(torch.autograd.Function):
    """(query, key, radius, max_neighbors) -> index; no gradients.
    Reference: torkit3d/ops/ball_query.py:6-14."""

    @staticmethod
    def forward(ctx, query, key, radius, max_neighbors, *extra):
        # extra (additions to the reference's signature): channel_first, index_dtype
        channel_first = bool(extra[0]) if len(extra) > 0 else False
        index_dtype = extra[1] if len(extra) > 1 else torch.int64
        cf, q, r = pick_layout(channel_first, query, key)
        index = _C.ball_query_cuda(q, r, radius, max_neighbors, channel_first=cf, index_dtype=index_dtype)
        ctx.mark_non_differentiable(index)
        ctx.n_args = 4 + len(extra)
        return index

    @staticmethod
    def backward(ctx, *grad_outputs):
        return _no_grads(ctx.n_args)


class GroupPointsFunction(torch.autograd.Function):
    """(points [B,C,N1], index [B,N2,K]) -> [B,C,N2,K]; saves index and N1.
    Reference: torkit3d/ops/group_points.py:6-19."""

    @staticmethod
    def forward(ctx, points, index, *extra):
        # extra (an addition to the reference's signature): rows = _C.feature_rows(points), built once
        # by a caller that groups the same features several times
        ctx.save_for_backward(index)
        ctx.num_points = points.size(2)
        ctx.n_extra = len(extra)
        if extra and extra[0] is not None:
            return _C.group_points_forward_rows_cuda(extra[0], index.contiguous())
        return _C.group_points_forward_cuda(points.contiguous(), index.contiguous())

    @staticmethod
    def backward(ctx, *grad_output):
        (index,) = ctx.saved_tensors
        grad_points = _C.group_points_backward_cuda(grad_output[0].contiguous(), index.contiguous(), ctx.num_points)
        return (grad_points, None) + _no_grads(ctx.n_extra)


class InterpolateFeature(torch.autograd.Function):
    """(feature [B,C,N1], index [B,N2,3], weight [B,N2,3]) -> [B,C,N2]; gradient for feature only.
    Reference: torkit3d/ops/interpolate_feature.py:6-24."""

    @staticmethod
    def forward(ctx, feature, index, weight, *extra):
        # extra (an addition to the reference's signature): rows = _C.feature_rows(feature), built once
        # by a caller that interpolates the same features several times (query slabs of one scene)
        ctx.save_for_backward(index, weight)
        ctx.n1 = feature.size(2)
        ctx.n_extra = len(extra)
        if extra and extra[0] is not None:
            return _C.interpolate_forward_rows_cuda(extra[0], index.contiguous(), weight.contiguous())
        return _C.interpolate_forward_cuda(feature.contiguous(), index.contiguous(), weight.contiguous())

    @staticmethod
    def backward(ctx, *grad_out):
        index, weight = ctx.saved_tensors
        grad_feature = _C.interpolate_backward_cuda(grad_out[0].contiguous(), index.contiguous(),
                                                    weight.contiguous(), ctx.n1)
        return (grad_feature, None, None) + _no_grads(ctx.n_extra)
