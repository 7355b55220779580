"""Edge features of EdgeConv (DGCNN): the data path of ``torkit3d/ops/edge_conv.py:46-97`` as one kernel."""
import torch

from .. import _fused


class EdgeFeatureFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query_feature, key_feature, key_ind, include_query):
        out = _fused.edge_feature_forward(query_feature, key_feature, key_ind, include_query)
        ctx.save_for_backward(key_ind)
        ctx.meta = (query_feature.size(1), key_feature.size(2), include_query)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (key_ind,) = ctx.saved_tensors
        C, n2, include_query = ctx.meta
        gq, gk = _fused.edge_feature_backward(grad_out, key_ind, C, n2, include_query,
                                              need_query=ctx.needs_input_grad[0], need_key=ctx.needs_input_grad[1])
        return gq, gk, None, None


def get_edge_feature(query_feature: torch.Tensor, key_feature: torch.Tensor, key_ind: torch.Tensor,
                     include_query: bool = True) -> torch.Tensor:
    """``cat([group_points(key_feature, key_ind) - query_feature[..., None], query_feature[..., None]], 1)``.

    Args:
        query_feature: [B, C, N1];  key_feature: [B, C, N2];  key_ind: [B, N1, K] int64.

    Returns:
        [B, 2C, N1, K] ([B, C, N1, K] without ``include_query``).
    """
    assert query_feature.size(0) == key_feature.size(0) == key_ind.size(0), [
        query_feature.size(0), key_feature.size(0), key_ind.size(0)]
    assert key_feature.size(1) == query_feature.size(1)
    assert key_ind.size(1) == query_feature.size(2)
    return EdgeFeatureFunction.apply(query_feature, key_feature, key_ind, bool(include_query))


get_edge_feature_custom = get_edge_feature
