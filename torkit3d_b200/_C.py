"""Drop-in for the reference's extension module ``torkit3d._C``.

Same nine functions, same argument order, same checks and the same ownership rule (the callee
allocates the outputs on the inputs' device) as ``torkit3d/csrc/torkit3d.cpp:13-21``; underneath,
each call goes through the C ABI of libtk3d_b200.so on the current CUDA stream of the tensors'
device.  float32 and float64 tensors are accepted, indices are int64.

Keyword-only extras (no counterpart in the reference, whose callers copy instead): the coordinate
operators take ``channel_first=True`` for [B,3,N] clouds, which are then read in place -- the
``.transpose(1, 2).contiguous()`` copy of torkit3d/ops/ball_query.py:32-36,
ops/sample_farthest_points.py:28-30, ops/knn_points.py:40-44 disappears -- and the index-producing
ones take ``index_dtype=torch.int32`` for half the index bytes.

Differences a caller can observe, all deliberate:
  * ``knn_distance_cuda`` returns every row sorted ascending by (distance, index); the reference
    leaves the row order unspecified.  ``version`` is validated (0 or 1) and otherwise ignored.
  * kernels are launched on the current stream of the tensors' device, not on the legacy default
    stream of whatever device happens to be current.
  * an out-of-range index in ``group_points`` / ``interpolate`` reads as 0 (forward) or is skipped
    (backward) instead of aborting the CUDA context with a device-side assert.
"""
import torch

from . import _lib
from ._lib import check, load


def _dtype(t):
    if t.dtype == torch.float32:
        return _lib.F32
    if t.dtype == torch.float64:
        return _lib.F64
    raise RuntimeError("tk3d: expected a float32 or float64 tensor, got %s" % t.dtype)


def _check_cuda_contig(**tensors):
    for name, t in tensors.items():
        if not t.is_cuda:
            raise RuntimeError("%s must be a CUDA tensor." % name)
        if not t.is_contiguous():
            raise RuntimeError("%s must be contiguous." % name)


def _check_cuda(**tensors):
    for name, t in tensors.items():
        if not t.is_cuda:
            raise RuntimeError("%s must be a CUDA tensor." % name)


def _check_eq(a, b, what):
    if a != b:
        raise RuntimeError("Check failed: %s (%d vs. %d)" % (what, a, b))


def _same_device_dtype(first, *rest, floats=()):
    for t in rest:
        if t.device != first.device:
            raise RuntimeError("tk3d: all tensors must be on the same device")
    for t in floats:
        if t.dtype != first.dtype:
            raise RuntimeError("tk3d: floating-point tensors must share one dtype")


def _index(t, name):
    if t.dtype != torch.int64:
        raise RuntimeError("%s must be an int64 tensor." % name)


def _index_code(index_dtype):
    if index_dtype == torch.int64:
        return _lib.I64
    if index_dtype == torch.int32:
        return _lib.I32
    raise RuntimeError("index_dtype must be torch.int64 or torch.int32, got %s" % (index_dtype,))


def _xyz_dims(channel_first):
    """(point axis, coordinate axis) of a cloud tensor."""
    return (2, 1) if channel_first else (1, 2)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t):
    """Handle of the current CUDA stream of the tensor's device (the raw getter avoids building a
    torch.cuda.Stream object per call)."""
    if _raw_stream is not None and t.device.index is not None:
        return _raw_stream(t.device.index)
    return torch.cuda.current_stream(t.device).cuda_stream


class _NoSwitch:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _on(device):
    """Context that makes ``device`` current; free when it already is (the usual case: the small
    operators are dominated by host time, and torch.cuda.device() costs several microseconds).
    The tensors at hand are CUDA tensors, so the runtime is initialised and the raw getter (a
    quarter of the cost of torch.cuda.current_device()) may be asked directly."""
    index = device.index
    if index is None or index == (_raw_device() if _raw_device is not None else torch.cuda.current_device()):
        return _NO_SWITCH
    return torch.cuda.device(device)


# Below this output size the forward gathers run without the transposed scratch copy: one launch
# instead of two (measured on B200: 16 MB of grouped output 0.039 ms with it, 0.020 ms without).
_ROWS_MIN_OUTPUT_BYTES = 48 << 20


def _ptr(t):
    return t.data_ptr()  # 0 for an empty tensor, which ctypes passes as NULL


def sample_farthest_points_cuda(points, num_samples, *, channel_first=False):
    """points [B,N,3] ([B,3,N] with ``channel_first``) -> index [B,num_samples] int64 (first sample is point 0)."""
    _check_cuda_contig(points=points)
    _check_eq(points.dim(), 3, "points.dim() == 3")
    pdim, cdim = _xyz_dims(channel_first)
    _check_eq(points.size(cdim), 3, "points.size(%d) == 3" % cdim)
    num_samples = int(num_samples)
    if not num_samples > 0:
        raise RuntimeError("Check failed: num_samples > 0 (%d vs. 0)" % num_samples)
    if not points.size(pdim) >= num_samples:
        raise RuntimeError("Check failed: points.size(%d) >= num_samples (%d vs. %d)"
                           % (pdim, points.size(pdim), num_samples))
    lib = load()
    B, N = points.size(0), points.size(pdim)
    dt = _dtype(points)
    with _on(points.device):
        index = torch.empty((B, num_samples), dtype=torch.int64, device=points.device)
        need = _lib.scratch_bytes("tk3d_fps", B, N, dt)
        scratch = torch.empty((need,), dtype=torch.uint8, device=points.device) if need else None
        if channel_first:
            check(lib.tk3d_fps_layout(_ptr(points), B, N, num_samples, 1, _ptr(index),
                                      _ptr(scratch) if need else None, need, dt, _stream(points)))
        else:
            check(lib.tk3d_fps(_ptr(points), B, N, num_samples, _ptr(index), _ptr(scratch) if need else None, need,
                               dt, _stream(points)))
    return index


def ball_query_cuda(query, key, radius, max_neighbors, *, channel_first=False, index_dtype=torch.int64):
    """query [B,N1,3], key [B,N2,3] ([B,3,N1], [B,3,N2] with ``channel_first``) -> index [B,N1,max_neighbors]."""
    _check_cuda_contig(query=query, key=key)
    _check_eq(query.dim(), 3, "query.dim() == 3")
    _check_eq(key.dim(), 3, "key.dim() == 3")
    _check_eq(query.size(0), key.size(0), "query.size(0) == key.size(0)")
    pdim, cdim = _xyz_dims(channel_first)
    _check_eq(query.size(cdim), 3, "query.size(%d) == 3" % cdim)
    _check_eq(key.size(cdim), 3, "key.size(%d) == 3" % cdim)
    _same_device_dtype(query, key, floats=(key,))
    lib = load()
    B, N1, N2 = query.size(0), query.size(pdim), key.size(pdim)
    k = int(max_neighbors)
    with _on(query.device):
        index = torch.empty((B, N1, k), dtype=index_dtype, device=query.device)
        if channel_first or index_dtype != torch.int64:
            check(lib.tk3d_ball_query_layout(_ptr(query), _ptr(key), B, N1, N2, float(radius), k,
                                             1 if channel_first else 0, _ptr(index), _index_code(index_dtype),
                                             _dtype(query), _stream(query)))
        else:
            check(lib.tk3d_ball_query(_ptr(query), _ptr(key), B, N1, N2, float(radius), k, _ptr(index),
                                      _dtype(query), _stream(query)))
    return index


def group_points_forward_cuda(input, index):
    """input [B,C,N1], index [B,N2,K] (int64, or int32 as an opt-in) -> [B,C,N2,K]."""
    si, sx = input.shape, index.shape
    if not (input.is_cuda and index.is_cuda and len(si) == 3 and len(sx) == 3 and si[0] == sx[0]
            and (index.dtype is torch.int64 or index.dtype is torch.int32) and input.device == index.device
            and input.is_contiguous() and index.is_contiguous()):
        _check_cuda(input=input, index=index)
        _check_eq(input.dim(), 3, "input.dim() == 3")
        _check_eq(index.dim(), 3, "index.dim() == 3")
        _check_eq(input.size(0), index.size(0), "input.size(0) == index.size(0)")
        if index.dtype not in (torch.int64, torch.int32):
            raise RuntimeError("index must be an int64 tensor.")
        _same_device_dtype(input, index)
        input, index = input.contiguous(), index.contiguous()
    lib = load()
    B, C, N1 = input.shape
    _, N2, K = index.shape
    with _on(input.device):
        out = torch.empty((B, C, N2, K), dtype=input.dtype, device=input.device)
        # the row-gather path (transpose into scratch, then gather) pays from about 48 MB of output on;
        # shapes the channel-row kernel serves report a scratch size of 0
        big = out.numel() * out.element_size() >= _ROWS_MIN_OUTPUT_BYTES
        need = _lib.scratch_bytes("tk3d_group_fwd", B, C, N1, N2, K, _dtype(input)) if big else 0
        scratch = torch.empty((need,), dtype=torch.uint8, device=input.device) if need else None
        if index.dtype == torch.int32:
            check(lib.tk3d_group_fwd_layout(_ptr(input), _ptr(index), _lib.I32, B, C, N1, N2, K, _ptr(out), None,
                                            _ptr(scratch) if need else None, need, _dtype(input), _stream(input)))
        else:
            check(lib.tk3d_group_fwd(_ptr(input), _ptr(index), B, C, N1, N2, K, _ptr(out), None,
                                     _ptr(scratch) if need else None, need, _dtype(input), _stream(input)))
    return out


def group_points_backward_cuda(grad_output, index, n1):
    """grad_output [B,C,N2,K], index [B,N2,K] -> grad_input [B,C,n1]."""
    sg, sx = grad_output.shape, index.shape
    if not (grad_output.is_cuda and index.is_cuda and len(sg) == 4 and len(sx) == 3 and sx[0] == sg[0]
            and sx[1] == sg[2] and sx[2] == sg[3] and index.dtype is torch.int64
            and grad_output.device == index.device and grad_output.is_contiguous() and index.is_contiguous()):
        _check_cuda_contig(grad_output=grad_output, index=index)
        _check_eq(grad_output.dim(), 4, "grad_output.dim() == 4")
        _check_eq(index.dim(), 3, "index.dim() == 3")
        _check_eq(index.size(0), grad_output.size(0), "index.size(0) == grad_output.size(0)")
        _check_eq(index.size(1), grad_output.size(2), "index.size(1) == grad_output.size(2)")
        _check_eq(index.size(2), grad_output.size(3), "index.size(2) == grad_output.size(3)")
        _index(index, "index")
        _same_device_dtype(grad_output, index)
    lib = load()
    B, C, N2, K = grad_output.shape
    n1 = int(n1)
    with _on(grad_output.device):
        gin = torch.empty((B, C, n1), dtype=grad_output.dtype, device=grad_output.device)
        need = _lib.scratch_bytes("tk3d_group_bwd", B, C, n1, N2, K, _dtype(grad_output))
        scratch = torch.empty((need,), dtype=torch.uint8, device=grad_output.device) if need else None
        check(lib.tk3d_group_bwd(_ptr(grad_output), _ptr(index), B, C, n1, N2, K, _ptr(gin), None,
                                 _ptr(scratch) if need else None, need, _dtype(grad_output), _stream(grad_output)))
    return gin


def _check_interp(a, index, weight, aname):
    # one combined test for the usual case (these operators are host-bound on small tensors); the
    # ordered checks below only run to produce the reference's message for what is wrong
    sa, si, sw = a.shape, index.shape, weight.shape
    if (a.is_cuda and index.is_cuda and weight.is_cuda and len(sa) == 3 and len(si) == 3 and len(sw) == 3
            and sa[0] == si[0] == sw[0] and si[1] == sw[1] and si[2] == 3 and sw[2] == 3
            and index.dtype is torch.int64 and weight.dtype is a.dtype and a.device == index.device == weight.device
            and a.is_contiguous() and index.is_contiguous() and weight.is_contiguous()):
        return
    _check_cuda_contig(**{aname: a, "index": index, "weight": weight})
    _check_eq(a.dim(), 3, aname + ".dim() == 3")
    _check_eq(index.dim(), 3, "index.dim() == 3")
    _check_eq(weight.dim(), 3, "weight.dim() == 3")
    _check_eq(a.size(0), index.size(0), aname + ".size(0) == index.size(0)")
    _check_eq(a.size(0), weight.size(0), aname + ".size(0) == weight.size(0)")
    _check_eq(index.size(1), weight.size(1), "index.size(1) == weight.size(1)")
    _check_eq(index.size(2), weight.size(2), "index.size(2) == weight.size(2)")
    if index.size(2) != 3:
        raise RuntimeError("Only support k=3.")
    _index(index, "index")
    _same_device_dtype(a, index, weight, floats=(weight,))


def interpolate_forward_cuda(input, index, weight):
    """input [B,C,N1], index/weight [B,N2,3] -> [B,C,N2]."""
    _check_interp(input, index, weight, "input")
    lib = load()
    B, C, N1 = input.shape
    N2 = index.size(1)
    with _on(input.device):
        out = torch.empty((B, C, N2), dtype=input.dtype, device=input.device)
        big = out.numel() * out.element_size() >= _ROWS_MIN_OUTPUT_BYTES
        need = _lib.scratch_bytes("tk3d_interp_fwd", B, C, N1, N2, _dtype(input)) if big else 0
        scratch = torch.empty((need,), dtype=torch.uint8, device=input.device) if need else None
        check(lib.tk3d_interp_fwd(_ptr(input), _ptr(index), _ptr(weight), B, C, N1, N2, 3, _ptr(out), None,
                                  _ptr(scratch) if need else None, need, _dtype(input), _stream(input)))
    return out


def interpolate_backward_cuda(grad_output, index, weight, n1):
    """grad_output [B,C,N2], index/weight [B,N2,3] -> grad_input [B,C,n1]."""
    _check_interp(grad_output, index, weight, "grad_output")
    _check_eq(grad_output.size(2), index.size(1), "grad_output.size(2) == index.size(1)")
    lib = load()
    B, C, N2 = grad_output.shape
    n1 = int(n1)
    with _on(grad_output.device):
        gin = torch.empty((B, C, n1), dtype=grad_output.dtype, device=grad_output.device)
        need = _lib.scratch_bytes("tk3d_interp_bwd", B, C, n1, N2, _dtype(grad_output))
        scratch = torch.empty((need,), dtype=torch.uint8, device=grad_output.device) if need else None
        check(lib.tk3d_interp_bwd(_ptr(grad_output), _ptr(index), _ptr(weight), B, C, n1, N2, 3, _ptr(gin), None,
                                  _ptr(scratch) if need else None, need, _dtype(grad_output), _stream(grad_output)))
    return gin


def feature_rows(feature):
    """feature [B,C,N] float32 -> the same values as rows [B,N,C]: the layout the row gathers read.
    Build it once when several gathers read the same features (query slabs of one scene, several
    groupings of one cloud) and pass it to the ``*_rows_cuda`` forms below.  No counterpart in the
    reference."""
    _check_cuda_contig(feature=feature)
    _check_eq(feature.dim(), 3, "feature.dim() == 3")
    if feature.dtype != torch.float32:
        raise RuntimeError("feature_rows: float32 features only")
    lib = load()
    B, C, N = feature.shape
    with _on(feature.device):
        rows = torch.empty((B, N, C), dtype=feature.dtype, device=feature.device)
        check(lib.tk3d_feature_rows(_ptr(feature), B, C, N, _ptr(rows), _lib.F32, _stream(feature)))
    return rows


def _check_rows(rows, index):
    _check_cuda_contig(rows=rows, index=index)
    _check_eq(rows.dim(), 3, "rows.dim() == 3")
    _check_eq(index.dim(), 3, "index.dim() == 3")
    _check_eq(rows.size(0), index.size(0), "rows.size(0) == index.size(0)")
    if rows.dtype != torch.float32:
        raise RuntimeError("rows must be a float32 tensor.")
    if index.dtype not in (torch.int64, torch.int32):
        raise RuntimeError("index must be an int64 tensor.")
    _same_device_dtype(rows, index)


def interpolate_forward_rows_cuda(rows, index, weight):
    """rows [B,N1,C] (``feature_rows`` of the [B,C,N1] features), index/weight [B,N2,3] -> [B,C,N2];
    the result of ``interpolate_forward_cuda`` on those features, without the per-call transposition."""
    _check_rows(rows, index)
    _check_cuda_contig(weight=weight)
    _check_eq(weight.dim(), 3, "weight.dim() == 3")
    _check_eq(index.size(1), weight.size(1), "index.size(1) == weight.size(1)")
    _check_eq(index.size(2), weight.size(2), "index.size(2) == weight.size(2)")
    if index.size(2) != 3:
        raise RuntimeError("Only support k=3.")
    _same_device_dtype(rows, weight, floats=(weight,))
    lib = load()
    B, N1, C = rows.shape
    N2 = index.size(1)
    with _on(rows.device):
        out = torch.empty((B, C, N2), dtype=rows.dtype, device=rows.device)
        check(lib.tk3d_interp_fwd_rows(_ptr(rows), _ptr(index), _index_code(index.dtype), _ptr(weight), B, C, N1, N2,
                                       3, _ptr(out), None, _lib.F32, _stream(rows)))
    return out


def group_points_forward_rows_cuda(rows, index):
    """rows [B,N1,C] (``feature_rows`` of the [B,C,N1] features), index [B,N2,K] -> [B,C,N2,K]."""
    _check_rows(rows, index)
    lib = load()
    B, N1, C = rows.shape
    _, N2, K = index.shape
    with _on(rows.device):
        out = torch.empty((B, C, N2, K), dtype=rows.dtype, device=rows.device)
        check(lib.tk3d_group_fwd_rows(_ptr(rows), _ptr(index), _index_code(index.dtype), B, C, N1, N2, K, _ptr(out),
                                      None, _lib.F32, _stream(rows)))
    return out


def knn_distance_cuda(query, key, k, version=0, *, channel_first=False, index_dtype=torch.int64):
    """query [B,N1,3], key [B,N2,3] ([B,3,N1], [B,3,N2] with ``channel_first``) ->
    [distance [B,N1,k] (squared), index [B,N1,k]]."""
    _check_cuda_contig(query=query, key=key)
    pdim, cdim = _xyz_dims(channel_first)
    _check_eq(query.dim(), 3, "query.dim() == 3")
    _check_eq(query.size(cdim), 3, "query.size(%d) == 3" % cdim)
    _check_eq(key.dim(), 3, "key.dim() == 3")
    _check_eq(key.size(0), query.size(0), "key.size(0) == query.size(0)")
    k = int(k)
    if not key.size(pdim) >= k:
        raise RuntimeError("Check failed: key.size(%d) >= k (%d vs. %d)" % (pdim, key.size(pdim), k))
    _check_eq(key.size(cdim), 3, "key.size(%d) == 3" % cdim)
    if version not in (0, 1):
        raise RuntimeError("Invalid version")
    _same_device_dtype(query, key, floats=(key,))
    lib = load()
    B, N1, N2 = query.size(0), query.size(pdim), key.size(pdim)
    with _on(query.device):
        distance = torch.empty((B, N1, k), dtype=query.dtype, device=query.device)
        index = torch.empty((B, N1, k), dtype=index_dtype, device=query.device)
        if channel_first or index_dtype != torch.int64:
            check(lib.tk3d_knn_layout(_ptr(query), _ptr(key), B, N1, N2, k, 1 if channel_first else 0,
                                      _ptr(distance), _ptr(index), _index_code(index_dtype), _dtype(query),
                                      _stream(query)))
        else:
            check(lib.tk3d_knn(_ptr(query), _ptr(key), B, N1, N2, k, _ptr(distance), _ptr(index), _dtype(query),
                               _stream(query)))
    return [distance, index]


def feature_knn_cuda(query, key, k, channel_first=True):
    """query [B,C,N1], key [B,C,N2] (or [B,N1,C], [B,N2,C] with ``channel_first=False``), float32 ->
    [distance [B,N1,k] (squared), index [B,N1,k] int64], rows sorted by (distance, index).

    No counterpart in the reference's extension: its models get these neighbours from
    ``torkit3d.ops.native.knn`` (cdist + topk, torkit3d/ops/native.py:4-30).
    """
    _check_cuda_contig(query=query, key=key)
    _check_eq(query.dim(), 3, "query.dim() == 3")
    _check_eq(key.dim(), 3, "key.dim() == 3")
    _check_eq(key.size(0), query.size(0), "key.size(0) == query.size(0)")
    cdim, ndim = (1, 2) if channel_first else (2, 1)
    _check_eq(key.size(cdim), query.size(cdim), "key channels == query channels")
    k = int(k)
    if not key.size(ndim) >= k:
        raise RuntimeError("Check failed: key.size(%d) >= k (%d vs. %d)" % (ndim, key.size(ndim), k))
    _same_device_dtype(query, key, floats=(key,))
    if query.dtype != torch.float32:
        raise RuntimeError("feature_knn_cuda: float32 tensors only")
    lib = load()
    B, C, N1, N2 = query.size(0), query.size(cdim), query.size(ndim), key.size(ndim)
    with _on(query.device):
        distance = torch.empty((B, N1, k), dtype=query.dtype, device=query.device)
        index = torch.empty((B, N1, k), dtype=torch.int64, device=query.device)
        check(lib.tk3d_feature_knn(_ptr(query), _ptr(key), B, C, N1, N2, k, 1 if channel_first else 0,
                                   _ptr(distance), _ptr(index), _dtype(query), _stream(query)))
    return [distance, index]


def chamfer_distance_forward_cuda(xyz1, xyz2, sums=None, *, channel_first=False):
    """xyz1 [B,N1,3], xyz2 [B,N2,3] ([B,3,N1], [B,3,N2] with ``channel_first``) -> [dist1, idx1, dist2, idx2].

    ``sums`` (optional, a float64 CUDA tensor of 2 elements) receives sum(dist1), sum(dist2); it has
    no counterpart in the reference and is what the multi-GPU loss helper reduces.
    """
    pdim, cdim = _xyz_dims(channel_first)
    s1, s2 = xyz1.shape, xyz2.shape
    # one combined test for the usual case; the ordered checks only run to name what is wrong
    if not (xyz1.is_cuda and xyz2.is_cuda and len(s1) == 3 and len(s2) == 3 and s1[0] == s2[0] and s1[cdim] == 3
            and s2[cdim] == 3 and xyz1.dtype is xyz2.dtype and xyz1.device == xyz2.device and xyz1.is_contiguous()
            and xyz2.is_contiguous()):
        _check_cuda_contig(xyz1=xyz1, xyz2=xyz2)
        _check_eq(xyz1.dim(), 3, "xyz1.dim() == 3")
        _check_eq(xyz2.dim(), 3, "xyz2.dim() == 3")
        _check_eq(xyz1.size(0), xyz2.size(0), "xyz1.size(0) == xyz2.size(0)")
        _check_eq(xyz1.size(cdim), 3, "xyz1.size(%d) == 3" % cdim)
        _check_eq(xyz2.size(cdim), 3, "xyz2.size(%d) == 3" % cdim)
        _same_device_dtype(xyz1, xyz2, floats=(xyz2,))
    lib = load()
    B, N1, N2 = s1[0], s1[pdim], s2[pdim]
    dev = xyz1.device
    with _on(dev):
        dist1 = torch.empty((B, N1), dtype=xyz1.dtype, device=dev)
        idx1 = torch.empty((B, N1), dtype=torch.int64, device=dev)
        dist2 = torch.empty((B, N2), dtype=xyz1.dtype, device=dev)
        idx2 = torch.empty((B, N2), dtype=torch.int64, device=dev)
        if sums is not None:
            if not (sums.is_cuda and sums.dtype == torch.float64 and sums.numel() == 2 and sums.is_contiguous()):
                raise RuntimeError("sums must be a contiguous float64 CUDA tensor with 2 elements")
        if channel_first:
            check(lib.tk3d_chamfer_fwd_layout(_ptr(xyz1), _ptr(xyz2), B, N1, N2, 1, _ptr(dist1), _ptr(idx1),
                                              _ptr(dist2), _ptr(idx2), _ptr(sums) if sums is not None else None,
                                              _dtype(xyz1), _stream(xyz1)))
        else:
            check(lib.tk3d_chamfer_fwd(_ptr(xyz1), _ptr(xyz2), B, N1, N2, _ptr(dist1), _ptr(idx1), _ptr(dist2),
                                       _ptr(idx2), _ptr(sums) if sums is not None else None, _dtype(xyz1),
                                       _stream(xyz1)))
    return [dist1, idx1, dist2, idx2]


def _chamfer_backward_checks(grad_dist1, grad_dist2, xyz1, xyz2, idx1, idx2, pdim, cdim):
    _check_cuda_contig(grad_dist1=grad_dist1, grad_dist2=grad_dist2, xyz1=xyz1, xyz2=xyz2, idx1=idx1, idx2=idx2)
    bs, n1, n2 = grad_dist1.size(0), grad_dist1.size(1), grad_dist2.size(1)
    _check_eq(grad_dist2.size(0), bs, "grad_dist2.size(0) == bs")
    _check_eq(xyz1.size(0), bs, "xyz1.size(0) == bs")
    _check_eq(xyz2.size(0), bs, "xyz2.size(0) == bs")
    _check_eq(xyz1.size(pdim), n1, "xyz1.size(%d) == n1" % pdim)
    _check_eq(xyz2.size(pdim), n2, "xyz2.size(%d) == n2" % pdim)
    _check_eq(xyz1.size(cdim), 3, "xyz1.size(%d) == 3" % cdim)
    _check_eq(xyz2.size(cdim), 3, "xyz2.size(%d) == 3" % cdim)
    _check_eq(idx1.size(0), bs, "idx1.size(0) == bs")
    _check_eq(idx2.size(0), bs, "idx2.size(0) == bs")
    _check_eq(idx1.size(1), n1, "idx1.size(1) == n1")
    _check_eq(idx2.size(1), n2, "idx2.size(1) == n2")
    _index(idx1, "idx1")
    _index(idx2, "idx2")
    _same_device_dtype(grad_dist1, grad_dist2, xyz1, xyz2, idx1, idx2, floats=(grad_dist2, xyz1, xyz2))


def chamfer_distance_backward_cuda(grad_dist1, grad_dist2, xyz1, xyz2, idx1, idx2, *, channel_first=False):
    """-> [grad_xyz1 [B,N1,3], grad_xyz2 [B,N2,3]] (the clouds' own layout: [B,3,N] with ``channel_first``)."""
    pdim, cdim = _xyz_dims(channel_first)
    sg1, sg2, s1, s2 = grad_dist1.shape, grad_dist2.shape, xyz1.shape, xyz2.shape
    ok = (len(sg1) == 2 and len(sg2) == 2 and len(s1) == 3 and len(s2) == 3 and idx1.shape == sg1 and idx2.shape == sg2
          and sg1[0] == sg2[0] == s1[0] == s2[0] and s1[pdim] == sg1[1] and s2[pdim] == sg2[1] and s1[cdim] == 3
          and s2[cdim] == 3 and idx1.dtype is torch.int64 and idx2.dtype is torch.int64
          and grad_dist1.dtype is grad_dist2.dtype is xyz1.dtype is xyz2.dtype
          and grad_dist1.is_cuda and grad_dist1.device == grad_dist2.device == xyz1.device == xyz2.device == idx1.device
          == idx2.device and grad_dist1.is_contiguous() and grad_dist2.is_contiguous() and xyz1.is_contiguous()
          and xyz2.is_contiguous() and idx1.is_contiguous() and idx2.is_contiguous())
    if not ok:  # the ordered checks name what is wrong, in the reference's words
        _chamfer_backward_checks(grad_dist1, grad_dist2, xyz1, xyz2, idx1, idx2, pdim, cdim)
    bs, n1, n2 = sg1[0], sg1[1], sg2[1]
    lib = load()
    dev = grad_dist1.device
    with _on(dev):
        g1 = torch.empty_like(xyz1)
        g2 = torch.empty_like(xyz2)
        if channel_first:
            check(lib.tk3d_chamfer_bwd_layout(_ptr(grad_dist1), _ptr(grad_dist2), _ptr(xyz1), _ptr(xyz2), _ptr(idx1),
                                              _ptr(idx2), bs, n1, n2, 1, _ptr(g1), _ptr(g2), _dtype(grad_dist1),
                                              _stream(grad_dist1)))
        else:
            check(lib.tk3d_chamfer_bwd(_ptr(grad_dist1), _ptr(grad_dist2), _ptr(xyz1), _ptr(xyz2), _ptr(idx1),
                                       _ptr(idx2), bs, n1, n2, _ptr(g1), _ptr(g2), _dtype(grad_dist1),
                                       _stream(grad_dist1)))
    return [g1, g2]


def three_nn_weight_cuda(distance):
    """Inverse squared-distance weights over the last axis; [.., k] -> [.., k] (k <= 8)."""
    _check_cuda_contig(distance=distance)
    lib = load()
    k = distance.size(-1)
    with _on(distance.device):
        w = torch.empty_like(distance)
        check(lib.tk3d_three_nn_weight(_ptr(distance), distance.numel() // max(k, 1), k, _ptr(w), _dtype(distance),
                                       _stream(distance)))
    return w
