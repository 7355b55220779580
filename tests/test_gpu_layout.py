"""Channel-first clouds read in place and 32-bit index outputs.

The reference's operators copy every [B,3,N] input with ``.transpose(1, 2).contiguous()`` before the
call (torkit3d/ops/ball_query.py:32-36, ops/sample_farthest_points.py:28-30, ops/knn_points.py:40-44,
ops/chamfer_distance.py:49-52).  The ``*_layout`` entry points read that tensor directly.  These tests
hold both layouts and both index types to the same results, element for element, over shapes that
reach every kernel behind the operators (fp32 fast paths, fp64 generic and split kernels, large k),
compare one case per operator with the CPU oracle, and check through the profiler that a
channel-first call launches no copy kernel.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def cf(t):
    """[B,N,3] -> dense [B,3,N]."""
    return t.transpose(1, 2).contiguous()


KNN_SHAPES = [(2, 100, 300, 3, torch.float32), (2, 700, 2000, 4, torch.float32), (4, 1000, 1111, 16, torch.float32),
              (40, 600, 700, 16, torch.float32), (2, 300, 2100, 32, torch.float32), (2, 257, 2200, 64, torch.float32),
              (1, 130, 4100, 128, torch.float32), (2, 50, 16, 16, torch.float32), (1, 64, 300, 200, torch.float32),
              (2, 300, 1300, 16, torch.float64), (1, 64, 300, 100, torch.float64), (200, 1000, 64, 8, torch.float64)]


@pytest.mark.parametrize("B,n1,n2,k,dt", KNN_SHAPES)
def test_knn_layouts_and_index_types(B, n1, n2, k, dt):
    from torkit3d_b200 import _C

    g = torch.Generator().manual_seed(n1 + k)
    q = torch.randn(B, n1, 3, generator=g, dtype=dt).to(DEV)
    r = torch.randn(B, n2, 3, generator=g, dtype=dt).to(DEV)
    d0, i0 = _C.knn_distance_cuda(q, r, k, 1)
    d1, i1 = _C.knn_distance_cuda(cf(q), cf(r), k, 1, channel_first=True)
    d2, i2 = _C.knn_distance_cuda(q, r, k, 1, index_dtype=torch.int32)
    d3, i3 = _C.knn_distance_cuda(cf(q), cf(r), k, 1, channel_first=True, index_dtype=torch.int32)
    assert i2.dtype == torch.int32 and i3.dtype == torch.int32 and i0.dtype == torch.int64
    for d, i in ((d1, i1), (d2, i2), (d3, i3)):
        assert torch.equal(d, d0)
        assert torch.equal(i.long(), i0)


BALL_SHAPES = [(2, 64, 128, 0.3, 32, torch.float32), (3, 65, 1290, 0.2, 16, torch.float32),
               (64, 3000, 1024, 0.25, 8, torch.float32), (3, 65, 129, 10.0, 32, torch.float32),
               (2, 100, 700, 0.3, 100, torch.float32), (2, 300, 900, 0.3, 24, torch.float64)]


@pytest.mark.parametrize("B,n1,n2,r,k,dt", BALL_SHAPES)
def test_ball_query_layouts_and_index_types(B, n1, n2, r, k, dt):
    from torkit3d_b200 import _C

    g = torch.Generator().manual_seed(n1 + k)
    key = torch.rand(B, n2, 3, generator=g, dtype=dt).to(DEV)
    query = torch.rand(B, n1, 3, generator=g, dtype=dt).to(DEV)
    i0 = _C.ball_query_cuda(query, key, r, k)
    i1 = _C.ball_query_cuda(cf(query), cf(key), r, k, channel_first=True)
    i2 = _C.ball_query_cuda(query, key, r, k, index_dtype=torch.int32)
    i3 = _C.ball_query_cuda(cf(query), cf(key), r, k, channel_first=True, index_dtype=torch.int32)
    assert i2.dtype == torch.int32 and i3.dtype == torch.int32
    for i in (i1, i2, i3):
        assert torch.equal(i.long(), i0)


@pytest.mark.parametrize("B,n,s,dt", [(2, 1024, 128, torch.float32), (2, 8192, 300, torch.float32),
                                      (1, 12000, 64, torch.float32), (1, 20000, 64, torch.float32),
                                      (3, 1025, 129, torch.float64), (1, 9000, 40, torch.float64)])
def test_fps_layouts(B, n, s, dt):
    from torkit3d_b200 import _C

    g = torch.Generator().manual_seed(n + s)
    p = torch.rand(B, n, 3, generator=g, dtype=dt).to(DEV)
    assert torch.equal(_C.sample_farthest_points_cuda(cf(p), s, channel_first=True),
                       _C.sample_farthest_points_cuda(p, s))


CHAMFER_SHAPES = [(2, 300, 257, torch.float32), (3, 4000, 3000, torch.float32), (24, 4096, 4096, torch.float32),
                  (1, 1, 5, torch.float32), (2, 200, 333, torch.float64)]


@pytest.mark.parametrize("B,n1,n2,dt", CHAMFER_SHAPES)
def test_chamfer_layouts_forward_and_backward(B, n1, n2, dt):
    from torkit3d_b200 import _C

    g = torch.Generator().manual_seed(n1 + n2)
    a = torch.randn(B, n1, 3, generator=g, dtype=dt).to(DEV)
    b = torch.randn(B, n2, 3, generator=g, dtype=dt).to(DEV)
    sums0 = torch.zeros(2, dtype=torch.float64, device=DEV)
    sums1 = torch.zeros(2, dtype=torch.float64, device=DEV)
    out0 = _C.chamfer_distance_forward_cuda(a, b, sums0)
    out1 = _C.chamfer_distance_forward_cuda(cf(a), cf(b), sums1, channel_first=True)
    for x, y in zip(out0, out1):
        assert torch.equal(x, y)
    torch.testing.assert_close(sums0, sums1, rtol=1e-12, atol=0)
    g1, g2 = torch.randn_like(out0[0]), torch.randn_like(out0[2])
    ga0, gb0 = _C.chamfer_distance_backward_cuda(g1, g2, a, b, out0[1], out0[3])
    ga1, gb1 = _C.chamfer_distance_backward_cuda(g1, g2, cf(a), cf(b), out0[1], out0[3], channel_first=True)
    assert ga1.shape == (B, 3, n1) and gb1.shape == (B, 3, n2)
    tol = dict(rtol=1e-5, atol=1e-6) if dt == torch.float32 else dict(rtol=1e-12, atol=1e-12)
    torch.testing.assert_close(ga1.transpose(1, 2), ga0, **tol)   # atomics reorder the scattered sums
    torch.testing.assert_close(gb1.transpose(1, 2), gb0, **tol)


def test_operators_pass_channel_first_tensors_through_without_a_copy(oracle):
    """ops.*(transpose=True) on dense [B,3,N] tensors: results equal the oracle's and the only kernels
    launched are the library's own (no PyTorch copy / element-wise kernel in the profile)."""
    from torch.profiler import ProfilerActivity, profile

    from torkit3d_b200.ops import ball_query, chamfer_distance, knn_points, sample_farthest_points

    rng = np.random.default_rng(5)
    p = rng.random((4, 2048, 3)).astype(np.float32)
    q = rng.random((4, 256, 3)).astype(np.float32)
    pcf, qcf = cf(T(p)), cf(T(q))
    torch.cuda.synchronize()

    def run():
        return (ball_query(qcf, pcf, 0.2, 16, transpose=True),
                sample_farthest_points(pcf, 64, transpose=True),
                knn_points(qcf, pcf, 8, transpose=True),
                chamfer_distance(qcf, pcf, transpose=True))

    run()  # warm-up (library load, allocator pools)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        ball, fps, (kd, ki), (c1, c2) = run()
        torch.cuda.synchronize()
    names = [e.key for e in prof.key_averages() if e.device_type == torch.autograd.DeviceType.CUDA]
    kernels = [n for n in names if "memset" not in n.lower() and "memcpy" not in n.lower()]
    assert kernels, "profiler saw no kernels"
    foreign = [n for n in kernels if "tk3d" not in n]
    assert not foreign, foreign
    assert not any("Memcpy" in n for n in names), names

    np.testing.assert_array_equal(ball.cpu().numpy(), oracle.ball_query(q, p, 0.2, 16))
    np.testing.assert_array_equal(fps.cpu().numpy(), oracle.fps(p, 64))
    ed, ei = oracle.knn(q, p, 8)
    np.testing.assert_array_equal(ki.cpu().numpy(), ei)
    np.testing.assert_array_equal(kd.cpu().numpy(), ed)
    e1, _, e2, _ = oracle.chamfer_fwd(q, p)
    np.testing.assert_array_equal(c1.cpu().numpy(), e1)
    np.testing.assert_array_equal(c2.cpu().numpy(), e2)


def test_transposed_views_go_through_without_a_copy_too():
    """A [B,N,3] tensor handed over as its [B,3,N] view (and the other way round) is recognised and read
    through its dense base; gradients come back in the caller's view."""
    from torkit3d_b200.ops import chamfer_distance, knn_points

    g = torch.Generator().manual_seed(9)
    a = torch.randn(2, 500, 3, generator=g).to(DEV).requires_grad_(True)
    b = torch.randn(2, 400, 3, generator=g).to(DEV).requires_grad_(True)
    d1, d2 = chamfer_distance(a, b)
    (d1.sum() + d2.sum()).backward()
    ga, gb = a.grad.clone(), b.grad.clone()
    a.grad = b.grad = None
    e1, e2 = chamfer_distance(a.transpose(1, 2), b.transpose(1, 2), transpose=True)   # views of dense [B,N,3]
    assert torch.equal(e1, d1) and torch.equal(e2, d2)
    (e1.sum() + e2.sum()).backward()
    torch.testing.assert_close(a.grad, ga, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(b.grad, gb, rtol=1e-5, atol=1e-6)
    acf = a.detach().transpose(1, 2).contiguous().requires_grad_(True)              # dense [B,3,N]
    bcf = b.detach().transpose(1, 2).contiguous().requires_grad_(True)
    f1, f2 = chamfer_distance(acf, bcf, transpose=True)
    assert torch.equal(f1, d1) and torch.equal(f2, d2)
    (f1.sum() + f2.sum()).backward()
    assert acf.grad.shape == acf.shape
    torch.testing.assert_close(acf.grad.transpose(1, 2), ga, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(bcf.grad.transpose(1, 2), gb, rtol=1e-5, atol=1e-6)
    k0 = knn_points(a.detach(), b.detach(), 5)
    k1 = knn_points(acf.detach().transpose(1, 2), bcf.detach().transpose(1, 2), 5)   # views of dense [B,3,N]
    assert torch.equal(k0[0], k1[0]) and torch.equal(k0[1], k1[1])


def test_layout_entry_points_reject_bad_index_dtype():
    from torkit3d_b200 import _lib

    lib = _lib.load()
    x = torch.zeros(1, 8, 3, device=DEV)
    i = torch.zeros(1, 8, 2, dtype=torch.int64, device=DEV)
    d = torch.zeros(1, 8, 2, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.tk3d_knn_layout(x.data_ptr(), x.data_ptr(), 1, 8, 8, 2, 0, d.data_ptr(), i.data_ptr(), 7, _lib.F32,
                               st) == 4
    assert lib.tk3d_ball_query_layout(x.data_ptr(), x.data_ptr(), 1, 8, 8, 0.5, 2, 1, i.data_ptr(), -1, _lib.F32,
                                      st) == 4


@pytest.mark.parametrize("B,C,n1,n2,k,dt", [(2, 16, 1024, 256, 16, torch.float32), (3, 7, 333, 50, 5, torch.float32),
                                            (2, 64, 300, 700, 32, torch.float32), (2, 8, 100, 40, 6, torch.float64)])
def test_group_points_reads_int32_indices(B, C, n1, n2, k, dt):
    """ball_query(index_dtype=int32) -> group_points without widening the index: same output as with int64."""
    from torkit3d_b200 import _C

    g = torch.Generator().manual_seed(n1 + k)
    f = torch.randn(B, C, n1, generator=g, dtype=dt).to(DEV)
    idx = torch.randint(0, n1, (B, n2, k), generator=g).to(DEV)
    out64 = _C.group_points_forward_cuda(f, idx)
    out32 = _C.group_points_forward_cuda(f, idx.int())
    assert torch.equal(out64, out32)
    assert torch.equal(out64, torch.gather(f.unsqueeze(2).expand(B, C, n2, n1), 3, idx.unsqueeze(1).expand(B, C, n2, k)))
