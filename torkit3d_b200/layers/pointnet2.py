"""Fused front ends of the PointNet++ modules.

What the reference spells as a chain of operator calls plus element-wise PyTorch glue is one call
here, over coordinates in the ``[B,3,N]`` layout its layers pass around:

===========================================  ===================================================
reference                                    here
===========================================  ===================================================
``sample_farthest_points(p, S, True)`` +     ``sample_and_gather(p, S)``
``batch_index_select(p, idx, dim=2)``
(models/classification/pointnet2.py:73-74)
``SetAbstraction.forward`` up to its MLP     ``set_abstraction_group(...)`` /
(layers/pointnet2.py:43-58, BallQuery)       ``SetAbstractionGrouper``
``FeatureInterpolator.forward``              ``three_nn_interpolate(...)`` /
(layers/pointnet2.py:114-133)                ``FeatureInterpolator``
===========================================  ===================================================

The MLPs, pooling and heads around them are ordinary ``torch.nn`` code and stay with the caller.
Gradients flow exactly where they do in the reference: into the features (and, for the grouping,
into both coordinate tensors through the centred xyz channels); neighbour search is not
differentiated.  Inputs the fused kernels do not serve (float64, k != 3, very wide features) take
the operator-by-operator route on the same GPU kernels the operators use.
"""
import torch
import torch.nn as nn

from .. import _fused
from ..ops.ball_query import ball_query
from ..ops.group_points import group_points
from ..ops.interpolate_feature import interpolate_feature
from ..ops.knn_points import knn_points


def sample_and_gather(points, num_samples):
    """points [B,3,N] -> (fps_index [B,S] int64, xyz_fps [B,3,S]); not differentiable w.r.t. index,
    xyz_fps carries the gradient of a gather."""
    index, sampled = _SampleAndGather.apply(points, int(num_samples))
    return index, sampled


class _SampleAndGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, points, num_samples):
        index, sampled = _fused.fps_gather(points, num_samples, channel_first=True)
        ctx.save_for_backward(index)
        ctx.n = points.size(2)
        ctx.mark_non_differentiable(index)
        return index, sampled

    @staticmethod
    def backward(ctx, _grad_index, grad_sampled):
        (index,) = ctx.saved_tensors
        grad = grad_sampled.new_zeros((grad_sampled.size(0), 3, ctx.n))
        grad.scatter_add_(2, index.unsqueeze(1).expand(-1, 3, -1), grad_sampled)
        return grad, None


class _SetAbstractionGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, in_xyz, out_xyz, in_feature, radius, max_neighbors, use_xyz):
        needs = ctx.needs_input_grad
        want_index = any(needs[:3])
        out, index32 = _fused.sa_group_forward(in_xyz, out_xyz, in_feature, radius, max_neighbors, use_xyz=use_xyz,
                                               channel_first=True, want_index=want_index)
        if want_index:
            ctx.save_for_backward(index32)
        ctx.meta = (0 if in_feature is None else in_feature.size(1), in_xyz.size(2), use_xyz)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (index32,) = ctx.saved_tensors
        C, N, use_xyz = ctx.meta
        needs = ctx.needs_input_grad
        gfeat, gpts, gcen = _fused.sa_group_backward(grad_out, index32, C, N, use_xyz=use_xyz, channel_first=True,
                                                     need_feature=needs[2], need_points=needs[0],
                                                     need_centroids=needs[1])
        return gpts, gcen, gfeat, None, None, None


def set_abstraction_group(in_xyz, out_xyz, in_feature, radius, max_neighbors, use_xyz=True):
    """Neighbourhood tensor that enters the shared MLP of a set-abstraction layer.

    Args:
        in_xyz: [B,3,N1] coordinates of the input points.
        out_xyz: [B,3,N2] coordinates of the group centres.
        in_feature: [B,C,N1] or None.
        radius, max_neighbors: ball-query parameters (K = max_neighbors).
        use_xyz: append the centred neighbour coordinates as 3 extra channels.

    Returns:
        [B, C(+3), N2, K]: ``cat([group_points(in_feature, idx), group_points(in_xyz, idx) -
        out_xyz[..., None]], 1)`` with ``idx = ball_query(out_xyz, in_xyz, radius, K)``.
    """
    assert in_xyz.size(0) == out_xyz.size(0)
    assert in_xyz.size(1) == out_xyz.size(1) == 3
    B, N1, N2 = in_xyz.size(0), in_xyz.size(2), out_xyz.size(2)
    C = 0 if in_feature is None else in_feature.size(1)
    if in_xyz.is_cuda and _fused.sa_group_supported(B, C, N1, N2, int(max_neighbors), in_xyz.dtype) and (
            in_feature is None or in_feature.dtype == torch.float32) and (C > 0 or use_xyz):
        return _SetAbstractionGroup.apply(in_xyz, out_xyz, in_feature, float(radius), int(max_neighbors),
                                          bool(use_xyz))
    # operator by operator
    with torch.no_grad():
        nbr_index = ball_query(out_xyz, in_xyz, radius, max_neighbors)
    parts = []
    if in_feature is not None:
        parts.append(group_points(in_feature, nbr_index))
    if use_xyz:
        parts.append(group_points(in_xyz, nbr_index) - out_xyz.unsqueeze(-1))
    if not parts:
        return in_xyz.new_empty([B, 0, nbr_index.size(1), nbr_index.size(2)])
    return parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)


class BallQuery(nn.Module):
    """Same constructor and call as the reference's module of this name (layers/pointnet2.py:71-85)."""

    def __init__(self, radius, max_neighbors):
        super().__init__()
        self.radius = radius
        self.max_neighbors = max_neighbors

    def forward(self, query, key):
        return ball_query(query, key, self.radius, self.max_neighbors)

    def extra_repr(self):
        return "radius={}, max_neighbors={}".format(self.radius, self.max_neighbors)


class SetAbstractionGrouper(nn.Module):
    """The parameter-free first half of ``SetAbstraction``: (in_xyz, out_xyz, in_feature) ->
    neighbourhood tensor [B, C(+3), N2, K].  ``query_neighbor`` is a ``BallQuery``."""

    def __init__(self, query_neighbor, use_xyz=True):
        super().__init__()
        self.query_neighbor = query_neighbor
        self.use_xyz = use_xyz

    def forward(self, in_xyz, out_xyz, in_feature):
        q = self.query_neighbor
        return set_abstraction_group(in_xyz, out_xyz, in_feature, q.radius, q.max_neighbors, self.use_xyz)

    def extra_repr(self):
        return "use_xyz={}".format(self.use_xyz)


class _ThreeNNInterpolate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query_xyz, key_xyz, key_feature, eps):
        out, index32, weight = _fused.three_nn_interp_forward(query_xyz, key_xyz, key_feature, eps=eps,
                                                              channel_first=True)
        ctx.save_for_backward(index32, weight)
        ctx.nk = key_xyz.size(2)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        index32, weight = ctx.saved_tensors
        gfeat = _fused.three_nn_interp_backward(grad_out, index32, weight, ctx.nk) if ctx.needs_input_grad[2] else None
        return None, None, gfeat, None


def three_nn_interpolate(query_xyz, key_xyz, key_feature, num_neighbors=3, eps=1e-10):
    """Inverse-distance interpolation of key features at the query points.

    Args:
        query_xyz: [B,3,N1];  key_xyz: [B,3,N2];  key_feature: [B,C,N2].

    Returns:
        [B,C,N1].  The reference's module of this purpose calls ``knn_points`` with its default
        ``transpose=False`` on ``[B,3,N]`` inputs, which fails the operator's shape check; here the
        channel-first layout is what the kernel reads.
    """
    fused = (num_neighbors == 3 and query_xyz.is_cuda and query_xyz.dtype == torch.float32
             and key_feature.dtype == torch.float32 and key_feature.size(1) <= 512 and key_xyz.size(2) >= 3
             and query_xyz.size(0) <= 65535)
    if fused:
        return _ThreeNNInterpolate.apply(query_xyz, key_xyz, key_feature, float(eps))
    with torch.no_grad():
        distance, index = knn_points(query_xyz, key_xyz, num_neighbors, transpose=True)
        inv_distance = 1.0 / torch.clamp(distance, min=eps)
        weight = inv_distance / torch.sum(inv_distance, dim=2, keepdim=True)
    return interpolate_feature(key_feature, index, weight)


class FeatureInterpolator(nn.Module):
    """Same constructor and call as the reference's module (layers/pointnet2.py:108-139)."""

    def __init__(self, num_neighbors=3, eps=1e-10):
        super().__init__()
        self.num_neighbors = num_neighbors
        self._eps = eps

    def forward(self, query_xyz, key_xyz, key_feature):
        return three_nn_interpolate(query_xyz, key_xyz, key_feature, self.num_neighbors, self._eps)

    def extra_repr(self):
        return "num_neighbors={}".format(self.num_neighbors)
