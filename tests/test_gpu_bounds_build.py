"""The range-checked build (-DTK3D_BOUNDS): the same entry points with every coordinate load and
index-tensor access checked against its tensor's extent.  A set of shapes that reaches every kernel
behind the coordinate operators runs through it; it must count no violation and return what the
regular build returns.  (CPU part: both libraries load, the regular one reports "no checks".)"""
import pytest
import torch

DEV = "cuda:0"


def test_regular_build_reports_no_checks_and_bounds_build_loads():
    from torkit3d_b200 import _lib

    assert _lib.load().tk3d_bounds_violations() == -1
    lib = _lib.load_bounds_checked()
    for name in _lib.SIGNATURES:
        assert hasattr(lib, name)


@pytest.mark.gpu
def test_bounds_build_counts_no_violation_and_matches_the_regular_build():
    from torkit3d_b200 import _lib

    reg, chk = _lib.load(), _lib.load_bounds_checked()
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(1)
    assert chk.tk3d_bounds_violations() == 0

    def both(fn):
        a = fn(reg)
        b = fn(chk)
        torch.cuda.synchronize()
        for x, y in zip(a, b):
            assert torch.equal(x, y)

    for (B, n1, n2, k, dt) in ((2, 300, 500, 3, torch.float32), (3, 1000, 1111, 16, torch.float32),
                               (2, 257, 2200, 64, torch.float32), (1, 130, 4100, 128, torch.float32),
                               (2, 50, 16, 16, torch.float32), (1, 64, 300, 200, torch.float32),
                               (2, 300, 1300, 16, torch.float64), (1, 64, 300, 100, torch.float64)):
        code = _lib.F32 if dt == torch.float32 else _lib.F64
        q = torch.randn(B, n1, 3, generator=g, dtype=dt).to(DEV)
        r = torch.randn(B, n2, 3, generator=g, dtype=dt).to(DEV)
        for cf in (0, 1):
            qq = q.transpose(1, 2).contiguous() if cf else q
            rr = r.transpose(1, 2).contiguous() if cf else r

            def knn(lib):
                d = torch.empty(B, n1, k, dtype=dt, device=DEV)
                i = torch.empty(B, n1, k, dtype=torch.int32, device=DEV)
                assert lib.tk3d_knn_layout(qq.data_ptr(), rr.data_ptr(), B, n1, n2, k, cf, d.data_ptr(), i.data_ptr(),
                                           _lib.I32, code, st) == 0
                return d, i

            def ball(lib):
                i = torch.empty(B, n1, 24, dtype=torch.int64, device=DEV)
                assert lib.tk3d_ball_query_layout(qq.data_ptr(), rr.data_ptr(), B, n1, n2, 0.7, 24, cf, i.data_ptr(),
                                                  _lib.I64, code, st) == 0
                return (i,)

            def chamfer(lib):
                d1 = torch.empty(B, n1, dtype=dt, device=DEV)
                d2 = torch.empty(B, n2, dtype=dt, device=DEV)
                i1 = torch.empty(B, n1, dtype=torch.int64, device=DEV)
                i2 = torch.empty(B, n2, dtype=torch.int64, device=DEV)
                assert lib.tk3d_chamfer_fwd_layout(qq.data_ptr(), rr.data_ptr(), B, n1, n2, cf, d1.data_ptr(),
                                                   i1.data_ptr(), d2.data_ptr(), i2.data_ptr(), None, code, st) == 0
                return d1, i1, d2, i2

            both(knn)
            both(ball)
            both(chamfer)
    # farthest point sampling: one block per cloud (registers / shared memory), a cluster of blocks
    # per cloud, the streaming kernel; ball query with more neighbours than one tile can give
    for (B, n, s, dt) in ((3, 1025, 129, torch.float32), (2, 6000, 50, torch.float32), (2, 9000, 100, torch.float32),
                          (2, 20000, 60, torch.float32),
                          (1, 70001, 30, torch.float32), (1, 140000, 12, torch.float32), (2, 3000, 70, torch.float64)):
        code = _lib.F32 if dt == torch.float32 else _lib.F64
        p = torch.rand(B, n, 3, generator=g, dtype=dt).to(DEV)
        for cf in (0, 1):
            pp = p.transpose(1, 2).contiguous() if cf else p

            def fps(lib):
                need = lib.tk3d_fps_scratch_bytes(B, n, code)
                scr = torch.empty(max(need, 1), dtype=torch.uint8, device=DEV)
                i = torch.empty(B, s, dtype=torch.int64, device=DEV)
                c = torch.empty((B, 3, s) if cf else (B, s, 3), dtype=dt, device=DEV)
                assert lib.tk3d_fps_gather(pp.data_ptr(), B, n, s, cf, i.data_ptr(), c.data_ptr(),
                                           scr.data_ptr() if need else None, need, code, st) == 0
                return i, c

            both(fps)
    q = torch.rand(2, 100, 3, generator=g).to(DEV)
    r = torch.rand(2, 2000, 3, generator=g).to(DEV)

    def wide_ball(lib):
        i = torch.empty(2, 100, 300, dtype=torch.int32, device=DEV)
        assert lib.tk3d_ball_query_layout(q.data_ptr(), r.data_ptr(), 2, 100, 2000, 0.5, 300, 0, i.data_ptr(), _lib.I32,
                                          _lib.F32, st) == 0
        return (i,)

    both(wide_ball)
    assert chk.tk3d_bounds_violations() == 0
