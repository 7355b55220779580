"""Tensor-level bindings of the fused layer front ends of libtk3d_b200.so (``include/tk3d.h``, last
section).  They have no counterpart in ``torkit3d._C``: each one replaces a chain of operator calls
and element-wise PyTorch expressions in ``torkit3d/layers/pointnet2.py`` and
``torkit3d/models/*/pointnet2.py``.  float32 CUDA tensors only; coordinates are ``[B,3,N]``
(``channel_first=True``, the layout those layers receive) or ``[B,N,3]``.
"""
import torch

from . import _lib
from ._C import _check_cuda, _check_eq, _on, _ptr, _stream
from ._lib import check, load


def _f32(**tensors):
    for name, t in tensors.items():
        if t is not None and t.dtype != torch.float32:
            raise RuntimeError("%s must be a float32 tensor (got %s)." % (name, t.dtype))


def _xyz_shape(t, channel_first, name):
    _check_eq(t.dim(), 3, "%s.dim() == 3" % name)
    _check_eq(t.size(1 if channel_first else 2), 3, "%s has 3 coordinates" % name)
    return t.size(0), t.size(2 if channel_first else 1)


def _scratch(nbytes, device):
    return torch.empty((nbytes,), dtype=torch.uint8, device=device) if nbytes else None


def fps_gather(points, num_samples, channel_first=True):
    """points [B,3,N] (or [B,N,3]) -> (index [B,S] int64, sampled [B,3,S] (or [B,S,3]))."""
    _check_cuda(points=points)
    points = points.contiguous()
    B, N = _xyz_shape(points, channel_first, "points")
    S = int(num_samples)
    if not 0 < S <= N:
        raise RuntimeError("Check failed: 0 < num_samples <= N (%d vs. %d)" % (S, N))
    if points.dtype == torch.float32:
        dt = _lib.F32
    elif points.dtype == torch.float64:
        dt = _lib.F64
    else:
        raise RuntimeError("points must be float32 or float64.")
    lib = load()
    with _on(points.device):
        index = torch.empty((B, S), dtype=torch.int64, device=points.device)
        sampled = torch.empty((B, 3, S) if channel_first else (B, S, 3), dtype=points.dtype, device=points.device)
        need = _lib.scratch_bytes("tk3d_fps", B, N, dt)
        scratch = _scratch(need, points.device)
        check(lib.tk3d_fps_gather(_ptr(points), B, N, S, 1 if channel_first else 0, _ptr(index), _ptr(sampled),
                                  _ptr(scratch) if need else None, need, dt, _stream(points)))
    return index, sampled


def sa_group_supported(B, C, N, M, K, dtype):
    return dtype == torch.float32 and bool(load().tk3d_sa_group_supported(B, C, N, M, K, _lib.F32))


def sa_group_forward(points, centroids, feature, radius, max_neighbors, use_xyz=True, channel_first=True,
                     want_index=True):
    """-> (out [B,C(+3),M,K], index32 [B,M,K] int32 or None).  ``feature`` may be None (C = 0)."""
    _check_cuda(points=points, centroids=centroids)
    _f32(points=points, centroids=centroids, feature=feature)
    points, centroids = points.contiguous(), centroids.contiguous()
    B, N = _xyz_shape(points, channel_first, "points")
    B2, M = _xyz_shape(centroids, channel_first, "centroids")
    _check_eq(B, B2, "points.size(0) == centroids.size(0)")
    C = 0
    if feature is not None:
        _check_cuda(feature=feature)
        feature = feature.contiguous()
        _check_eq(feature.dim(), 3, "feature.dim() == 3")
        _check_eq(feature.size(0), B, "feature.size(0) == points.size(0)")
        _check_eq(feature.size(2), N, "feature.size(2) == number of points")
        C = feature.size(1)
    K = int(max_neighbors)
    lib = load()
    dev = points.device
    with _on(dev):
        out = torch.empty((B, C + (3 if use_xyz else 0), M, K), dtype=torch.float32, device=dev)
        index32 = torch.empty((B, M, K), dtype=torch.int32, device=dev) if want_index else None
        need = _lib.scratch_bytes("tk3d_sa_group", B, C, N, M, K, _lib.F32)
        scratch = _scratch(need, dev)
        check(lib.tk3d_sa_group_fwd(_ptr(points), _ptr(centroids), _ptr(feature) if C else None, B, C, N, M,
                                    float(radius), K, 1 if channel_first else 0, 1 if use_xyz else 0, _ptr(out),
                                    _ptr(index32) if want_index else None, None, _ptr(scratch) if need else None,
                                    need, _lib.F32, _stream(points)))
    return out, index32


def sa_group_backward(grad_out, index32, C, N, use_xyz=True, channel_first=True, need_feature=True, need_points=False,
                      need_centroids=False):
    """-> (grad_feature [B,C,N] | None, grad_points | None, grad_centroids | None)."""
    _check_cuda(grad_out=grad_out, index32=index32)
    _f32(grad_out=grad_out)
    grad_out = grad_out.contiguous()
    B, M, K = index32.shape
    _check_eq(grad_out.size(1), C + (3 if use_xyz else 0), "grad_out channels")
    lib = load()
    dev = grad_out.device
    with _on(dev):
        gfeat = torch.empty((B, C, N), dtype=torch.float32, device=dev) if (need_feature and C) else None
        xyz = use_xyz and (need_points or need_centroids)
        gpts = torch.empty((B, 3, N) if channel_first else (B, N, 3), dtype=torch.float32, device=dev) \
            if (xyz and need_points) else None
        gcen = torch.empty((B, 3, M) if channel_first else (B, M, 3), dtype=torch.float32, device=dev) \
            if (xyz and need_centroids) else None
        need = _lib.scratch_bytes("tk3d_sa_group", B, C, N, M, K, _lib.F32) if gfeat is not None else 0
        scratch = _scratch(need, dev)
        check(lib.tk3d_sa_group_bwd(_ptr(grad_out), _ptr(index32), B, C, N, M, K, 1 if channel_first else 0,
                                    1 if use_xyz else 0, _ptr(gfeat) if gfeat is not None else None,
                                    _ptr(gpts) if gpts is not None else None,
                                    _ptr(gcen) if gcen is not None else None, None,
                                    _ptr(scratch) if need else None, need, _lib.F32, _stream(grad_out)))
    return gfeat, gpts, gcen


def three_nn_interp_forward(query_xyz, key_xyz, key_feature, eps=1e-10, channel_first=True):
    """-> (out [B,C,Nq], index32 [B,Nq,3] int32, weight [B,Nq,3])."""
    _check_cuda(query_xyz=query_xyz, key_xyz=key_xyz, key_feature=key_feature)
    _f32(query_xyz=query_xyz, key_xyz=key_xyz, key_feature=key_feature)
    query_xyz, key_xyz, key_feature = query_xyz.contiguous(), key_xyz.contiguous(), key_feature.contiguous()
    B, Nq = _xyz_shape(query_xyz, channel_first, "query_xyz")
    B2, Nk = _xyz_shape(key_xyz, channel_first, "key_xyz")
    _check_eq(B, B2, "query_xyz.size(0) == key_xyz.size(0)")
    _check_eq(key_feature.dim(), 3, "key_feature.dim() == 3")
    _check_eq(key_feature.size(0), B, "key_feature.size(0) == key_xyz.size(0)")
    _check_eq(key_feature.size(2), Nk, "key_feature.size(2) == number of keys")
    C = key_feature.size(1)
    lib = load()
    dev = query_xyz.device
    with _on(dev):
        out = torch.empty((B, C, Nq), dtype=torch.float32, device=dev)
        index32 = torch.empty((B, Nq, 3), dtype=torch.int32, device=dev)
        weight = torch.empty((B, Nq, 3), dtype=torch.float32, device=dev)
        need = _lib.scratch_bytes("tk3d_three_nn_interp", B, C, Nq, Nk, _lib.F32)
        scratch = _scratch(need, dev)
        check(lib.tk3d_three_nn_interp_fwd(_ptr(query_xyz), _ptr(key_xyz), _ptr(key_feature), B, C, Nq, Nk,
                                           1 if channel_first else 0, float(eps), _ptr(out), _ptr(index32),
                                           _ptr(weight), None, _ptr(scratch) if need else None, need, _lib.F32,
                                           _stream(query_xyz)))
    return out, index32, weight


def three_nn_interp_backward(grad_out, index32, weight, Nk):
    """-> grad_feature [B,C,Nk]."""
    _check_cuda(grad_out=grad_out, index32=index32, weight=weight)
    _f32(grad_out=grad_out, weight=weight)
    grad_out = grad_out.contiguous()
    B, C, Nq = grad_out.shape
    lib = load()
    dev = grad_out.device
    with _on(dev):
        gfeat = torch.empty((B, C, Nk), dtype=torch.float32, device=dev)
        need = _lib.scratch_bytes("tk3d_three_nn_interp", B, C, Nq, Nk, _lib.F32)
        scratch = _scratch(need, dev)
        check(lib.tk3d_three_nn_interp_bwd(_ptr(grad_out), _ptr(index32), _ptr(weight), B, C, Nq, Nk, _ptr(gfeat),
                                           None, _ptr(scratch) if need else None, need, _lib.F32,
                                           _stream(grad_out)))
    return gfeat


def edge_feature_forward(query_feature, key_feature, index, include_query=True):
    """query_feature [B,C,N1], key_feature [B,C,N2], index [B,N1,K] int64 -> [B,2C,N1,K] (or [B,C,N1,K])."""
    from ._C import _dtype, _index

    _check_cuda(query_feature=query_feature, key_feature=key_feature, index=index)
    _index(index, "index")
    if query_feature.dtype != key_feature.dtype:
        raise RuntimeError("query_feature and key_feature must share one dtype.")
    query_feature, key_feature, index = query_feature.contiguous(), key_feature.contiguous(), index.contiguous()
    _check_eq(query_feature.dim(), 3, "query_feature.dim() == 3")
    _check_eq(key_feature.dim(), 3, "key_feature.dim() == 3")
    _check_eq(index.dim(), 3, "index.dim() == 3")
    B, C, N1 = query_feature.shape
    _check_eq(key_feature.size(0), B, "key_feature.size(0) == query_feature.size(0)")
    _check_eq(index.size(0), B, "index.size(0) == query_feature.size(0)")
    _check_eq(key_feature.size(1), C, "key_feature.size(1) == query_feature.size(1)")
    _check_eq(index.size(1), N1, "index.size(1) == query_feature.size(2)")
    N2, K = key_feature.size(2), index.size(2)
    dt = _dtype(query_feature)
    lib = load()
    dev = query_feature.device
    with _on(dev):
        out = torch.empty((B, 2 * C if include_query else C, N1, K), dtype=query_feature.dtype, device=dev)
        need = _lib.scratch_bytes("tk3d_edge_feature", B, C, N1, N2, K, dt)
        scratch = _scratch(need, dev)
        check(lib.tk3d_edge_feature_fwd(_ptr(query_feature), _ptr(key_feature), _ptr(index), B, C, N1, N2, K,
                                        1 if include_query else 0, _ptr(out), None,
                                        _ptr(scratch) if need else None, need, dt, _stream(query_feature)))
    return out


def edge_feature_backward(grad_out, index, C, N2, include_query=True, need_query=True, need_key=True):
    """-> (grad_query [B,C,N1] | None, grad_key [B,C,N2] | None)."""
    from ._C import _dtype

    _check_cuda(grad_out=grad_out, index=index)
    grad_out, index = grad_out.contiguous(), index.contiguous()
    B, N1, K = index.shape
    dt = _dtype(grad_out)
    lib = load()
    dev = grad_out.device
    with _on(dev):
        gq = torch.empty((B, C, N1), dtype=grad_out.dtype, device=dev) if need_query else None
        gk = torch.empty((B, C, N2), dtype=grad_out.dtype, device=dev) if need_key else None
        need = _lib.scratch_bytes("tk3d_edge_feature", B, C, N1, N2, K, dt) if need_key else 0
        scratch = _scratch(need, dev)
        check(lib.tk3d_edge_feature_bwd(_ptr(grad_out), _ptr(index), B, C, N1, N2, K, 1 if include_query else 0,
                                        _ptr(gq) if need_query else None, _ptr(gk) if need_key else None, None,
                                        _ptr(scratch) if need else None, need, dt, _stream(grad_out)))
    return gq, gk
