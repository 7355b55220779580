"""TEST INFRASTRUCTURE ONLY -- numpy front end of the CPU oracle (libtk3d_oracle.so).

Only tests/, the smoke check and the CPU-baseline leg of bench.py may import this module.  The
product package never does: it fails loudly when its CUDA library is missing.

Every function takes and returns numpy arrays (float32 or float64, int64 indices) in the layouts of
the reference extension (``torkit3d/csrc/torkit3d.cpp:13-21``).  Work is split over batch entries
on a thread pool (ctypes releases the GIL), so ``threads`` > 1 helps when B > 1.
"""
import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libtk3d_oracle.so")
_lib = None


def build(force=False):
    """Compile the oracle with gcc (-ffp-contract=off); a no-op when the library is up to date."""
    srcs = [os.path.join(_HERE, f) for f in ("tk3d_oracle.c", "tk3d_oracle_impl.h")]
    if (not force and os.path.exists(_SO)
            and all(os.path.getmtime(_SO) >= os.path.getmtime(s) for s in srcs if os.path.exists(s))):
        return _SO
    subprocess.run(["make", "-C", _HERE, "-B", "libtk3d_oracle.so"], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _sfx(a):
    if a.dtype == np.float32:
        return "_f32"
    if a.dtype == np.float64:
        return "_f64"
    raise TypeError("oracle supports float32/float64, got %s" % a.dtype)


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _c(a, dtype=None):
    return np.ascontiguousarray(a, dtype=dtype)


I64 = ctypes.c_int64


def _pool(n, threads, fn):
    """Run fn(b0, b1) over batch ranges on a thread pool."""
    threads = max(1, min(threads or (os.cpu_count() or 1), n))
    if threads == 1 or n <= 1:
        fn(0, n)
        return
    bounds = np.linspace(0, n, threads + 1).astype(int)
    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(lambda i: fn(int(bounds[i]), int(bounds[i + 1])), range(threads)))


def chamfer_fwd(xyz1, xyz2, threads=None):
    xyz1, xyz2 = _c(xyz1), _c(xyz2)
    B, N1, _ = xyz1.shape
    N2 = xyz2.shape[1]
    d1 = np.empty((B, N1), xyz1.dtype)
    i1 = np.empty((B, N1), np.int64)
    d2 = np.empty((B, N2), xyz1.dtype)
    i2 = np.empty((B, N2), np.int64)
    f = getattr(lib(), "orc_chamfer_fwd" + _sfx(xyz1))

    def run(b0, b1):
        if b1 > b0:
            f(_p(xyz1[b0:b1]), _p(xyz2[b0:b1]), I64(b1 - b0), I64(N1), I64(N2),
              _p(d1[b0:b1]), _p(i1[b0:b1]), _p(d2[b0:b1]), _p(i2[b0:b1]))

    _pool(B, threads, run)
    return d1, i1, d2, i2


def chamfer_bwd(g1, g2, xyz1, xyz2, idx1, idx2, threads=None):
    xyz1, xyz2 = _c(xyz1), _c(xyz2)
    g1, g2 = _c(g1, xyz1.dtype), _c(g2, xyz1.dtype)
    idx1, idx2 = _c(idx1, np.int64), _c(idx2, np.int64)
    B, N1, _ = xyz1.shape
    N2 = xyz2.shape[1]
    o1 = np.empty_like(xyz1)
    o2 = np.empty_like(xyz2)
    f = getattr(lib(), "orc_chamfer_bwd" + _sfx(xyz1))

    def run(b0, b1):
        if b1 > b0:
            f(_p(g1[b0:b1]), _p(g2[b0:b1]), _p(xyz1[b0:b1]), _p(xyz2[b0:b1]), _p(idx1[b0:b1]),
              _p(idx2[b0:b1]), I64(b1 - b0), I64(N1), I64(N2), _p(o1[b0:b1]), _p(o2[b0:b1]))

    _pool(B, threads, run)
    return o1, o2


def knn(query, key, k, threads=None):
    """Squared distances and indices, each row sorted ascending by (distance, index)."""
    query, key = _c(query), _c(key)
    B, N1, _ = query.shape
    N2 = key.shape[1]
    assert N2 >= k
    d = np.empty((B, N1, k), query.dtype)
    i = np.empty((B, N1, k), np.int64)
    f = getattr(lib(), "orc_knn" + _sfx(query))

    def run(b0, b1):
        if b1 > b0:
            f(_p(query[b0:b1]), _p(key[b0:b1]), I64(b1 - b0), I64(N1), I64(N2), I64(k), _p(d[b0:b1]), _p(i[b0:b1]))

    _pool(B, threads, run)
    return d, i


def feature_knn(query, key, k, channel_first=True, threads=None):
    """KNN on C-dimensional features: squared distances (fma over the channels in order) and
    indices, rows sorted ascending by (distance, index).  [B, C, N] tensors, or [B, N, C] with
    ``channel_first=False``."""
    query, key = _c(query), _c(key)
    B = query.shape[0]
    C, N1 = (query.shape[1], query.shape[2]) if channel_first else (query.shape[2], query.shape[1])
    N2 = key.shape[2] if channel_first else key.shape[1]
    assert N2 >= k
    d = np.empty((B, N1, k), query.dtype)
    i = np.empty((B, N1, k), np.int64)
    f = getattr(lib(), "orc_feature_knn" + _sfx(query))

    def run(b0, b1):
        if b1 > b0:
            f(_p(query[b0:b1]), _p(key[b0:b1]), I64(b1 - b0), I64(C), I64(N1), I64(N2), I64(k),
              ctypes.c_int(1 if channel_first else 0), _p(d[b0:b1]), _p(i[b0:b1]))

    _pool(B, threads, run)
    return d, i


def fps(points, num_samples, threads=None):
    points = _c(points)
    B, N, _ = points.shape
    out = np.empty((B, num_samples), np.int64)
    f = getattr(lib(), "orc_fps" + _sfx(points))

    def run(b0, b1):
        if b1 > b0:
            f(_p(points[b0:b1]), I64(b1 - b0), I64(N), I64(num_samples), _p(out[b0:b1]))

    _pool(B, threads, run)
    return out


def ball_query(query, key, radius, k, threads=None):
    query, key = _c(query), _c(key)
    B, N1, _ = query.shape
    N2 = key.shape[1]
    out = np.empty((B, N1, k), np.int64)
    f = getattr(lib(), "orc_ball_query" + _sfx(query))

    def run(b0, b1):
        if b1 > b0:
            f(_p(query[b0:b1]), _p(key[b0:b1]), I64(b1 - b0), I64(N1), I64(N2), ctypes.c_float(radius), I64(k),
              _p(out[b0:b1]))

    _pool(B, threads, run)
    return out


def group_fwd(inp, index, threads=None):
    inp, index = _c(inp), _c(index, np.int64)
    B, C, N1 = inp.shape
    _, N2, K = index.shape
    out = np.empty((B, C, N2, K), inp.dtype)
    f = getattr(lib(), "orc_group_fwd" + _sfx(inp))

    def run(b0, b1):
        if b1 > b0:
            f(_p(inp[b0:b1]), _p(index[b0:b1]), I64(b1 - b0), I64(C), I64(N1), I64(N2), I64(K), _p(out[b0:b1]))

    _pool(B, threads, run)
    return out


def group_bwd(gout, index, n1, threads=None):
    gout, index = _c(gout), _c(index, np.int64)
    B, C, N2, K = gout.shape
    out = np.empty((B, C, n1), gout.dtype)
    f = getattr(lib(), "orc_group_bwd" + _sfx(gout))

    def run(b0, b1):
        if b1 > b0:
            f(_p(gout[b0:b1]), _p(index[b0:b1]), I64(b1 - b0), I64(C), I64(n1), I64(N2), I64(K), _p(out[b0:b1]))

    _pool(B, threads, run)
    return out


def interp_fwd(inp, index, weight, threads=None):
    inp, index = _c(inp), _c(index, np.int64)
    weight = _c(weight, inp.dtype)
    B, C, N1 = inp.shape
    _, N2, K = index.shape
    out = np.empty((B, C, N2), inp.dtype)
    f = getattr(lib(), "orc_interp_fwd" + _sfx(inp))

    def run(b0, b1):
        if b1 > b0:
            f(_p(inp[b0:b1]), _p(index[b0:b1]), _p(weight[b0:b1]), I64(b1 - b0), I64(C), I64(N1), I64(N2), I64(K),
              _p(out[b0:b1]))

    _pool(B, threads, run)
    return out


def interp_bwd(gout, index, weight, n1, threads=None):
    gout, index = _c(gout), _c(index, np.int64)
    weight = _c(weight, gout.dtype)
    B, C, N2 = gout.shape
    K = index.shape[2]
    out = np.empty((B, C, n1), gout.dtype)
    f = getattr(lib(), "orc_interp_bwd" + _sfx(gout))

    def run(b0, b1):
        if b1 > b0:
            f(_p(gout[b0:b1]), _p(index[b0:b1]), _p(weight[b0:b1]), I64(b1 - b0), I64(C), I64(n1), I64(N2), I64(K),
              _p(out[b0:b1]))

    _pool(B, threads, run)
    return out


def three_nn_weight(dist):
    """Inverse squared-distance weights over the last axis (torkit3d/layers/pointnet2.py:128-130)."""
    dist = _c(dist)
    k = dist.shape[-1]
    out = np.empty_like(dist)
    getattr(lib(), "orc_three_nn_weight" + _sfx(dist))(_p(dist), I64(dist.size // k), I64(k), _p(out))
    return out


# ---- callers of the operators (compositions, numpy) ------------------------------------------------
def _group_safe(x, index):
    """group_points with -1 entries (empty ball-query rows) reading as 0: [B,C,N],[B,M,K] -> [B,C,M,K]."""
    safe = np.where(index < 0, 0, index)
    out = np.stack([x[b][:, safe[b]] for b in range(x.shape[0])])
    return np.where((index >= 0)[:, None], out, 0).astype(x.dtype)


def fps_gather(points_cf, num_samples):
    """sample_farthest_points(points, S, transpose=True) + batch_index_select(points, idx, dim=2)
    (torkit3d/models/classification/pointnet2.py:73-74).  points_cf [B,3,N] -> (idx [B,S], xyz [B,3,S])."""
    pts = np.ascontiguousarray(points_cf.transpose(0, 2, 1))
    idx = fps(pts, num_samples)
    xyz = np.take_along_axis(points_cf, np.broadcast_to(idx[:, None, :], (idx.shape[0], 3, idx.shape[1])), axis=2)
    return idx, xyz


def sa_group(in_xyz_cf, out_xyz_cf, feature, radius, k, use_xyz=True):
    """The tensor entering the MLP of SetAbstraction.forward (torkit3d/layers/pointnet2.py:43-58) with a
    BallQuery neighbour search: [B, C(+3), N2, K]."""
    pts = np.ascontiguousarray(in_xyz_cf.transpose(0, 2, 1))
    cen = np.ascontiguousarray(out_xyz_cf.transpose(0, 2, 1))
    index = ball_query(cen, pts, radius, k)
    parts = []
    if feature is not None:
        parts.append(_group_safe(feature, index))
    if use_xyz:
        parts.append((_group_safe(in_xyz_cf, index) - out_xyz_cf[..., None]).astype(in_xyz_cf.dtype))
    return np.concatenate(parts, axis=1), index


def edge_feature(query_feature, key_feature, index, include_query=True):
    """get_edge_feature_custom (torkit3d/ops/edge_conv.py:73-93): [B,2C,N1,K] (or [B,C,N1,K])."""
    grouped = _group_safe(key_feature, index)
    qe = np.broadcast_to(query_feature[..., None], grouped.shape)
    edge = (grouped - qe).astype(query_feature.dtype)
    return np.concatenate([edge, qe], axis=1) if include_query else edge


def three_nn_interp(query_cf, key_cf, key_feature, eps=1e-10):
    """FeatureInterpolator.forward (torkit3d/layers/pointnet2.py:114-133) on channel-first coordinates:
    -> (out [B,C,Nq] in float64 accumulation, index [B,Nq,3], weight [B,Nq,3])."""
    q = np.ascontiguousarray(query_cf.transpose(0, 2, 1))
    r = np.ascontiguousarray(key_cf.transpose(0, 2, 1))
    d, idx = knn(q, r, 3)
    one = d.dtype.type(1.0)
    inv = (one / np.maximum(d, d.dtype.type(eps))).astype(d.dtype)
    norm = ((inv[..., 0] + inv[..., 1]).astype(d.dtype) + inv[..., 2]).astype(d.dtype)
    w = (inv / norm[..., None]).astype(d.dtype)
    out = interp_fwd(key_feature.astype(np.float64), idx, w.astype(np.float64))
    return out, idx, w
