"""Guard bands around every output of the C ABI.

Each output (and scratch) buffer is carved out of a larger allocation whose surrounding bytes hold a
sentinel; after the call the bands must be untouched and every element inside must have been written
(the buffers start out as 0xEE bytes, which no result produces).  This catches writes outside a
tensor and elements an entry point forgets -- the library's contract is "every output element is
written by the call", so callers allocate with ``torch.empty``.  The reference's only run-time checks on
this path are device-side asserts on gather indices (torkit3d/csrc/cuda/group_points_kernel.cu:62,
interpolate_kernel.cu:40,141).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BAND = 4096          # bytes on either side
FILL = 0xEE


class Banded:
    """A tensor view with guard bands on both sides."""

    def __init__(self, shape, dtype):
        self.n = int(torch.tensor(shape).prod().item()) if len(shape) else 1
        self.nbytes = self.n * torch.empty((), dtype=dtype).element_size()
        pad = (-self.nbytes) % 16
        self.raw = torch.full((BAND + self.nbytes + pad + BAND,), FILL, dtype=torch.uint8, device=DEV)
        self.view = self.raw[BAND:BAND + self.nbytes].view(dtype).view(shape)

    def ptr(self):
        return self.view.data_ptr()

    def check(self, name, written=True):
        lo, hi = self.raw[:BAND], self.raw[BAND + self.nbytes:]
        assert bool((lo == FILL).all()) and bool((hi == FILL).all()), "%s: a guard band was written" % name
        if written and self.nbytes:
            body = self.raw[BAND:BAND + self.nbytes].view(-1, self.view.element_size())
            untouched = (body == FILL).all(dim=1)
            assert not bool(untouched.any()), "%s: %d elements were never written" % (name, int(untouched.sum()))


def _lib():
    from torkit3d_b200 import _lib

    return _lib, _lib.load()


def _st():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("B,n1,n2,dt", [(3, 1000, 777, torch.float32), (2, 4100, 4099, torch.float32), (2, 129, 65, torch.float64)])
@pytest.mark.parametrize("cf", [0, 1])
def test_chamfer_forward_backward(B, n1, n2, dt, cf):
    L, lib = _lib()
    code = L.F32 if dt == torch.float32 else L.F64
    shape1, shape2 = ((B, 3, n1), (B, 3, n2)) if cf else ((B, n1, 3), (B, n2, 3))
    a, b = torch.randn(shape1, dtype=dt, device=DEV), torch.randn(shape2, dtype=dt, device=DEV)
    d1, d2 = Banded((B, n1), dt), Banded((B, n2), dt)
    i1, i2 = Banded((B, n1), torch.int64), Banded((B, n2), torch.int64)
    sums = Banded((2,), torch.float64)
    assert lib.tk3d_chamfer_fwd_layout(a.data_ptr(), b.data_ptr(), B, n1, n2, cf, d1.ptr(), i1.ptr(), d2.ptr(), i2.ptr(),
                                       sums.ptr(), code, _st()) == 0
    torch.cuda.synchronize()
    for t, nm in ((d1, "dist1"), (d2, "dist2"), (i1, "idx1"), (i2, "idx2"), (sums, "sums")):
        t.check(nm)
    g1, g2 = torch.randn(B, n1, dtype=dt, device=DEV), torch.randn(B, n2, dtype=dt, device=DEV)
    ga, gb = Banded(shape1, dt), Banded(shape2, dt)
    assert lib.tk3d_chamfer_bwd_layout(g1.data_ptr(), g2.data_ptr(), a.data_ptr(), b.data_ptr(), i1.ptr(), i2.ptr(), B,
                                       n1, n2, cf, ga.ptr(), gb.ptr(), code, _st()) == 0
    torch.cuda.synchronize()
    ga.check("grad_xyz1")
    gb.check("grad_xyz2")


@pytest.mark.parametrize("B,n1,n2,k,dt", [(2, 300, 500, 3, torch.float32), (3, 1000, 1111, 16, torch.float32),
                                          (2, 257, 2200, 64, torch.float32), (2, 50, 16, 16, torch.float32),
                                          (1, 64, 300, 200, torch.float32), (2, 300, 1300, 16, torch.float64),
                                          (1, 64, 300, 100, torch.float64)])
@pytest.mark.parametrize("i32", [0, 1])
def test_knn(B, n1, n2, k, dt, i32):
    L, lib = _lib()
    code = L.F32 if dt == torch.float32 else L.F64
    q, r = torch.randn(B, n1, 3, dtype=dt, device=DEV), torch.randn(B, n2, 3, dtype=dt, device=DEV)
    d, i = Banded((B, n1, k), dt), Banded((B, n1, k), torch.int32 if i32 else torch.int64)
    assert lib.tk3d_knn_layout(q.data_ptr(), r.data_ptr(), B, n1, n2, k, 0, d.ptr(), i.ptr(), L.I32 if i32 else L.I64,
                               code, _st()) == 0
    torch.cuda.synchronize()
    d.check("distance")
    i.check("index")
    assert int(i.view.min()) >= 0 and int(i.view.max()) < n2


@pytest.mark.parametrize("B,n,s,dt", [(3, 1025, 129, torch.float32), (2, 9000, 100, torch.float32),
                                      (1, 20000, 50, torch.float32), (2, 1025, 129, torch.float64),
                                      (1, 9000, 40, torch.float64)])
def test_fps_and_gather(B, n, s, dt):
    L, lib = _lib()
    code = L.F32 if dt == torch.float32 else L.F64
    p = torch.rand(B, n, 3, dtype=dt, device=DEV)
    need = lib.tk3d_fps_scratch_bytes(B, n, code)
    idx, smp, scr = Banded((B, s), torch.int64), Banded((B, s, 3), dt), Banded((max(need, 1),), torch.uint8)
    assert lib.tk3d_fps_gather(p.data_ptr(), B, n, s, 0, idx.ptr(), smp.ptr(), scr.ptr() if need else None, need, code,
                               _st()) == 0
    torch.cuda.synchronize()
    idx.check("index")
    smp.check("sampled")
    scr.check("scratch", written=False)


@pytest.mark.parametrize("B,n1,n2,r,k,dt", [(3, 65, 1290, 0.2, 16, torch.float32), (64, 3000, 1024, 0.25, 8, torch.float32),
                                            (2, 100, 700, 0.3, 100, torch.float32), (2, 300, 900, 0.3, 24, torch.float64)])
@pytest.mark.parametrize("i32", [0, 1])
def test_ball_query(B, n1, n2, r, k, dt, i32):
    L, lib = _lib()
    code = L.F32 if dt == torch.float32 else L.F64
    q, key = torch.rand(B, n1, 3, dtype=dt, device=DEV), torch.rand(B, n2, 3, dtype=dt, device=DEV)
    i = Banded((B, n1, k), torch.int32 if i32 else torch.int64)
    assert lib.tk3d_ball_query_layout(q.data_ptr(), key.data_ptr(), B, n1, n2, r, k, 0, i.ptr(), L.I32 if i32 else L.I64,
                                      code, _st()) == 0
    torch.cuda.synchronize()
    i.check("index")
    assert int(i.view.min()) >= -1 and int(i.view.max()) < n2


@pytest.mark.parametrize("B,C,n1,n2,k", [(2, 64, 1024, 256, 16), (3, 7, 333, 50, 5), (2, 64, 300, 700, 32), (2, 33, 129, 100, 9)])
def test_group_and_interpolate(B, C, n1, n2, k):
    L, lib = _lib()
    f = torch.randn(B, C, n1, device=DEV)
    idx = torch.randint(0, n1, (B, n2, k), device=DEV)
    need = lib.tk3d_group_fwd_scratch_bytes(B, C, n1, n2, k, L.F32)
    out, scr = Banded((B, C, n2, k), torch.float32), Banded((max(need, 1),), torch.uint8)
    assert lib.tk3d_group_fwd(f.data_ptr(), idx.data_ptr(), B, C, n1, n2, k, out.ptr(), None, scr.ptr() if need else None,
                              need, L.F32, _st()) == 0
    go = torch.randn(B, C, n2, k, device=DEV)
    needb = lib.tk3d_group_bwd_scratch_bytes(B, C, n1, n2, k, L.F32)
    gin, scrb = Banded((B, C, n1), torch.float32), Banded((max(needb, 1),), torch.uint8)
    assert lib.tk3d_group_bwd(go.data_ptr(), idx.data_ptr(), B, C, n1, n2, k, gin.ptr(), None,
                              scrb.ptr() if needb else None, needb, L.F32, _st()) == 0
    idx3 = torch.randint(0, n1, (B, n2, 3), device=DEV)
    w = torch.rand(B, n2, 3, device=DEV)
    need3 = lib.tk3d_interp_fwd_scratch_bytes(B, C, n1, n2, L.F32)
    o3, scr3 = Banded((B, C, n2), torch.float32), Banded((max(need3, 1),), torch.uint8)
    assert lib.tk3d_interp_fwd(f.data_ptr(), idx3.data_ptr(), w.data_ptr(), B, C, n1, n2, 3, o3.ptr(), None,
                               scr3.ptr() if need3 else None, need3, L.F32, _st()) == 0
    g3 = torch.randn(B, C, n2, device=DEV)
    need3b = lib.tk3d_interp_bwd_scratch_bytes(B, C, n1, n2, L.F32)
    gi3, scr3b = Banded((B, C, n1), torch.float32), Banded((max(need3b, 1),), torch.uint8)
    assert lib.tk3d_interp_bwd(g3.data_ptr(), idx3.data_ptr(), w.data_ptr(), B, C, n1, n2, 3, gi3.ptr(), None,
                               scr3b.ptr() if need3b else None, need3b, L.F32, _st()) == 0
    torch.cuda.synchronize()
    for t, nm, wr in ((out, "group out", True), (scr, "group scratch", False), (gin, "group grad", True),
                      (scrb, "group bwd scratch", False), (o3, "interp out", True), (scr3, "interp scratch", False),
                      (gi3, "interp grad", True), (scr3b, "interp bwd scratch", False)):
        t.check(nm, written=wr)


@pytest.mark.parametrize("B,C,n1,n2,k", [(2, 64, 1024, 256, 16), (3, 7, 333, 50, 5), (2, 128, 4100, 9000, 3), (1, 512, 64, 40, 16)])
@pytest.mark.parametrize("i32", [0, 1])
def test_features_kept_as_rows(B, C, n1, n2, k, i32):
    L, lib = _lib()
    f = torch.randn(B, C, n1, device=DEV)
    rows = Banded((B, n1, C), torch.float32)
    assert lib.tk3d_feature_rows(f.data_ptr(), B, C, n1, rows.ptr(), L.F32, _st()) == 0
    it = torch.int32 if i32 else torch.int64
    code = L.I32 if i32 else L.I64
    idx = torch.randint(0, n1, (B, n2, k), device=DEV).to(it)
    out = Banded((B, C, n2, k), torch.float32)
    assert lib.tk3d_group_fwd_rows(rows.ptr(), idx.data_ptr(), code, B, C, n1, n2, k, out.ptr(), None, L.F32, _st()) == 0
    idx3 = torch.randint(0, n1, (B, n2, 3), device=DEV).to(it)
    w = torch.rand(B, n2, 3, device=DEV)
    o3 = Banded((B, C, n2), torch.float32)
    assert lib.tk3d_interp_fwd_rows(rows.ptr(), idx3.data_ptr(), code, w.data_ptr(), B, C, n1, n2, 3, o3.ptr(), None,
                                    L.F32, _st()) == 0
    torch.cuda.synchronize()
    rows.check("rows")
    out.check("group out")
    o3.check("interp out")
    assert torch.equal(rows.view, f.transpose(1, 2).contiguous())
