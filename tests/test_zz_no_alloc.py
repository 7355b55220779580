"""Farthest point sampling through the entry point that allocates nothing.

Who needs it: a host that may not allocate device memory at the place where it samples -- code
inside a region where its framework forbids allocation, a plugin with a memory budget fixed at
start-up, a plain-C caller without an allocator.  ``tk3d_fps_static_scratch`` keeps the running
minimum distances in an 8 MiB array built into the library instead of a caller buffer.

The test drives it through the C ABI, twice in a row on different inputs (the array keeps the
previous call's contents, which must not leak into the next result), and compares every index
with the regular entry point ``tk3d_fps`` fed with a caller-allocated scratch buffer and with the
CPU oracle (for large clouds both entry points run the same streaming kernel, so the oracle is the
independent check).  Indices are integers, so the comparisons are exact.  Device memory is watched
through the driver's free-memory figure, which also sees allocations made outside PyTorch.  This
file sorts last on purpose: a run that stops at the first failure has then already gone through
every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _regular(lib, points, S, dt):
    B, N, _ = points.shape
    idx = torch.full((B, S), -7, dtype=torch.int64, device=points.device)
    need = lib.tk3d_fps_scratch_bytes(B, N, dt)
    scratch = torch.empty(max(need, 1), dtype=torch.uint8, device=points.device)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.tk3d_fps(points.data_ptr(), B, N, S, idx.data_ptr(), scratch.data_ptr() if need else None, need, dt, st) == 0
    return idx


def _static(lib, points, S, dt):
    B, N, _ = points.shape
    idx = torch.full((B, S), -7, dtype=torch.int64, device=points.device)
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.tk3d_fps_static_scratch(points.data_ptr(), B, N, S, idx.data_ptr(), dt, st)
    assert rc == 0, lib.tk3d_last_error()
    return idx


def test_static_scratch_matches_regular_entry_point_twice_in_a_row(oracle):
    from torkit3d_b200 import _lib

    lib = _lib.load()
    assert lib.tk3d_fps_static_scratch_capacity() == 8 << 20
    g = torch.Generator().manual_seed(11)
    # 1st call: large clouds (the regular entry point needs scratch for these as well)
    p1 = torch.rand(3, 20000, 3, generator=g).to(DEV)
    # 2nd call: different shape and values, fp64, reusing the same built-in array
    p2 = (torch.rand(5, 3000, 3, generator=g, dtype=torch.float64) * 4 - 2).to(DEV)
    # 3rd call: small fp32 clouds, where the regular entry point keeps everything on chip
    p3 = torch.randn(4, 1500, 3, generator=g).to(DEV)
    # warm-up call: the first call on a device looks up the array's address (and loads the module)
    _static(lib, p3, 4, _lib.F32)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    got1 = _static(lib, p1, 96, _lib.F32)
    got2 = _static(lib, p2, 200, _lib.F64)
    got3 = _static(lib, p3, 300, _lib.F32)
    torch.cuda.synchronize()
    # only the three small index outputs were allocated (by this test), nothing the size of a scratch array
    assert torch.cuda.memory_allocated() - before < 64 * 1024
    # the driver's view: nothing near the size of a scratch array (8 MiB) was taken by anyone during
    # the three calls; PyTorch may add one 2 MiB segment to its pool for the index outputs
    assert free_before - torch.cuda.mem_get_info()[0] < (4 << 20)
    for got, pts, S, dt in ((got1, p1, 96, _lib.F32), (got2, p2, 200, _lib.F64), (got3, p3, 300, _lib.F32)):
        want = _regular(lib, pts, S, dt)
        assert torch.equal(got, want)
        assert np.array_equal(got.cpu().numpy(), oracle.fps(pts.cpu().numpy(), S))
        assert (got[:, 0] == 0).all() and (got >= 0).all() and (got < pts.size(1)).all()
    # same inputs again: identical output (nothing left over from the calls in between)
    assert torch.equal(_static(lib, p1, 96, _lib.F32), got1)


def test_static_scratch_rejects_sizes_beyond_the_built_in_array():
    from torkit3d_b200 import _lib

    lib = _lib.load()
    cap = lib.tk3d_fps_static_scratch_capacity()
    st = torch.cuda.current_stream().cuda_stream
    n_too_many = cap // 4 + 1
    pts = torch.zeros(1, 8, 3, device=DEV)  # never read: the size check comes first
    idx = torch.zeros(1, 4, dtype=torch.int64, device=DEV)
    assert lib.tk3d_fps_static_scratch(pts.data_ptr(), 1, n_too_many, 4, idx.data_ptr(), _lib.F32, st) == 6
    assert b"built-in scratch" in lib.tk3d_last_error()
    assert lib.tk3d_fps_static_scratch(pts.data_ptr(), 2, cap // 8, 4, idx.data_ptr(), _lib.F64, st) == 6
    # exactly at the limit is accepted
    n_max = cap // 4
    big = torch.rand(1, n_max, 3, device=DEV)
    out = torch.empty(1, 3, dtype=torch.int64, device=DEV)
    assert lib.tk3d_fps_static_scratch(big.data_ptr(), 1, n_max, 3, out.data_ptr(), _lib.F32, st) == 0
    assert torch.equal(out, _regular(lib, big, 3, _lib.F32))
    # the usual argument errors
    assert lib.tk3d_fps_static_scratch(pts.data_ptr(), 1, 8, 9, idx.data_ptr(), _lib.F32, st) == 3
    assert lib.tk3d_fps_static_scratch(None, 1, 8, 4, idx.data_ptr(), _lib.F32, st) == 1
