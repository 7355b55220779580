"""CUDA-graph capture of the launch-bound chains: the small chamfer configuration (forward +
backward) and the set-abstraction front end (FPS + centroid gather -> fused grouping).  A captured
graph is replayed on new input values written into the captured buffers and must reproduce what
the eager calls return for those values."""
import numpy as np
import pytest
import torch

from torkit3d_b200 import _C, _fused, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_graph_chamfer_c1():
    x1, x2 = workloads.c1_chamfer_small()
    a, b = x1.to(DEV), x2.to(DEV)
    g1 = torch.full((a.size(0), a.size(1)), 1e-3, device=DEV)
    g2 = torch.full((b.size(0), b.size(1)), 1e-3, device=DEV)

    def chain():
        d1, i1, d2, i2 = _C.chamfer_distance_forward_cuda(a, b)
        ga, gb = _C.chamfer_distance_backward_cuda(g1, g2, a, b, i1, i2)
        return d1, i1, d2, i2, ga, gb

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            chain()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = chain()
    # new values in the captured input buffers
    gen = torch.Generator().manual_seed(123)
    a.copy_(torch.rand(a.shape, generator=gen))
    b.copy_(torch.rand(b.shape, generator=gen))
    graph.replay()
    torch.cuda.synchronize()
    got = [o.clone() for o in outs]
    want = chain()
    for g, w in zip(got[:4], want[:4]):
        assert torch.equal(g, w)
    for g, w in zip(got[4:], want[4:]):
        torch.testing.assert_close(g, w, rtol=1e-5, atol=1e-6)


def test_graph_set_abstraction_front_end():
    p, feat = workloads.c3_set_abstraction(B=4, N=2048, C=32)
    pts = p.transpose(1, 2).contiguous().to(DEV)
    f = feat.to(DEV)

    def chain():
        index, cen = _fused.fps_gather(pts, 256)
        out, _ = _fused.sa_group_forward(pts, cen, f, 0.2, 32, want_index=False)
        return index, out

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            chain()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = chain()
    p2, feat2 = workloads.c3_set_abstraction(B=4, N=2048, C=32, seed=99)
    pts.copy_(p2.transpose(1, 2))
    f.copy_(feat2)
    graph.replay()
    torch.cuda.synchronize()
    got = [o.clone() for o in outs]
    want = chain()
    assert torch.equal(got[0], want[0])
    assert torch.equal(got[1], want[1])


def test_graph_large_k_small_ball_and_large_cloud_fps():
    """The kernels with several phases or a cluster launch inside one call -- radix-selection KNN
    (histogram sweeps, vote, collect, sort), the hit-mask ball query for few queries and the
    cluster FPS of a cloud beyond one block -- captured WITHOUT a warm-up call of these shapes
    before the capture (the first call of a kernel may raise its shared-memory limit or opt into
    the large cluster size while capturing), then replayed on new values."""
    gen = torch.Generator().manual_seed(321)
    q = torch.randn(2, 300, 3, generator=gen).to(DEV)
    r = torch.randn(2, 3000, 3, generator=gen).to(DEV)
    big = torch.rand(1, 70000, 3, generator=gen).to(DEV)
    mid = torch.rand(2, 7000, 3, generator=gen).to(DEV)  # clusters of eight small blocks, mbarriers in shared memory

    def chain():
        d, i = _C.knn_distance_cuda(q, r, 150, 0)
        bq = _C.ball_query_cuda(q, r, 0.6, 100)
        fp = _C.sample_farthest_points_cuda(big, 40)
        fm = _C.sample_farthest_points_cuda(mid, 90)
        return d, i, bq, fp, fm

    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = chain()
    for _ in range(2):
        q.copy_(torch.randn(q.shape, generator=gen))
        r.copy_(torch.randn(r.shape, generator=gen))
        big.copy_(torch.rand(big.shape, generator=gen))
        mid.copy_(torch.rand(mid.shape, generator=gen))
        graph.replay()
        torch.cuda.synchronize()
        got = [o.clone() for o in outs]
        want = chain()
        for g, w in zip(got, want):
            assert torch.equal(g, w)
