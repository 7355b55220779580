"""The sharded forms of the operators against the unsharded ones, on the GPU kernels.

Every rank of a multi-GPU run computes its shard with exactly the calls below (a batch shard for
chamfer / KNN / FPS / ball query / grouping, a query slab with keys and features replicated for the
scene-scale interpolation), so running the shards of every world size one after another on one GPU
and comparing their concatenation with the unsharded result checks what a 2-, 4- or 8-GPU run
produces, kernel dispatch included: a shard is smaller than the whole and may take another kernel
(fewer queries -> more warps per query, smaller outputs -> another gather path).  The reference
has no multi-GPU path; its operators are per-cloud and per-query independent
(torkit3d/csrc/cuda/knn_distance_kernel.cu:12-99, interpolate_kernel.cu:8-47).
"""
import pytest
import torch

from torkit3d_b200 import workloads
from torkit3d_b200.dist import batch_shard, chamfer_step, query_slab

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_scene_interpolation_by_query_slabs(world):
    from torkit3d_b200.ops import feature_rows, interpolate_feature, knn_points, three_nn_weight

    q, r, f = workloads.c5_scene_interp(B=2, NQ=40000, NR=9000, C=32)
    q, r, f = q.to(DEV), r.to(DEV), f.to(DEV)
    d, i = knn_points(q, r, 3)
    w = three_nn_weight(d)
    whole = interpolate_feature(f, i, w)
    rows = feature_rows(f)
    ds, idx, outs, outs_rows = [], [], [], []
    for rank in range(world):
        qs = query_slab(q, rank, world).contiguous()
        dr, ir = knn_points(qs, r, 3)
        wr = three_nn_weight(dr)
        ds.append(dr)
        idx.append(ir)
        outs.append(interpolate_feature(f, ir, wr))
        outs_rows.append(interpolate_feature(f, ir, wr, rows=rows))
    assert torch.equal(torch.cat(idx, 1), i)
    assert torch.equal(torch.cat(ds, 1), d)
    torch.testing.assert_close(torch.cat(outs, 2), whole, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(torch.cat(outs_rows, 2), whole, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_batch_shards(world):
    from torkit3d_b200.ops import ball_query, group_points, knn_points, sample_farthest_points

    x1, x2 = workloads.c4_chamfer_large(B=8, N=3000, M=2500, seed=5)
    a, b = x1.to(DEV), x2.to(DEV)
    loss, ga, gb = chamfer_step(a, b)
    parts = [chamfer_step(batch_shard(a, rk, world).contiguous(), batch_shard(b, rk, world).contiguous(),
                          global_batch=8) for rk in range(world)]
    # every rank holds the global mean only after the all-reduce; here: the shards' partial sums
    # are what that all-reduce adds, so the gradients (which need the counts only) must agree
    torch.testing.assert_close(torch.cat([p[1] for p in parts], 0), ga, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(torch.cat([p[2] for p in parts], 0), gb, rtol=1e-5, atol=1e-6)

    d, i = knn_points(a, b, 16)
    s = sample_farthest_points(a, 200)
    cent = torch.gather(a, 1, s.unsqueeze(-1).expand(-1, -1, 3)).contiguous()
    bq = ball_query(cent, a, 0.2, 24, transpose=False)
    feat = torch.randn(8, 16, 3000, device=DEV)
    gp = group_points(feat, bq.clamp(min=0))
    di, ii, ss, bb, gg = [], [], [], [], []
    for rk in range(world):
        ar, br = batch_shard(a, rk, world).contiguous(), batch_shard(b, rk, world).contiguous()
        dr, ir = knn_points(ar, br, 16)
        sr = sample_farthest_points(ar, 200)
        cr = torch.gather(ar, 1, sr.unsqueeze(-1).expand(-1, -1, 3)).contiguous()
        br_ = ball_query(cr, ar, 0.2, 24, transpose=False)
        di.append(dr)
        ii.append(ir)
        ss.append(sr)
        bb.append(br_)
        gg.append(group_points(batch_shard(feat, rk, world).contiguous(), br_.clamp(min=0)))
    assert torch.equal(torch.cat(ii, 0), i) and torch.equal(torch.cat(di, 0), d)
    assert torch.equal(torch.cat(ss, 0), s) and torch.equal(torch.cat(bb, 0), bq)
    assert torch.equal(torch.cat(gg, 0), gp)


def test_sharded_loss_is_the_sum_of_the_shards():
    """What the all-reduce adds up: the per-shard sums of distances, taken from the forward kernel's
    epilogue, against the unsharded batch (float64 sums: equal to 1e-12)."""
    from torkit3d_b200 import _C

    x1, x2 = workloads.c4_chamfer_large(B=8, N=2000, M=2000, seed=6)
    a, b = x1.to(DEV), x2.to(DEV)
    whole = torch.zeros(2, dtype=torch.float64, device=DEV)
    _C.chamfer_distance_forward_cuda(a, b, sums=whole)
    for world in (2, 4, 8):
        acc = torch.zeros(2, dtype=torch.float64, device=DEV)
        for rk in range(world):
            part = torch.zeros(2, dtype=torch.float64, device=DEV)
            _C.chamfer_distance_forward_cuda(batch_shard(a, rk, world).contiguous(),
                                             batch_shard(b, rk, world).contiguous(), sums=part)
            acc += part
        torch.testing.assert_close(acc, whole, rtol=1e-12, atol=0)
