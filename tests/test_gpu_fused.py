"""Fused layer front ends (FPS + centroid gather, set-abstraction grouping, three-NN
interpolation) against the CPU oracle's operators composed the way the reference's layers compose
them (torkit3d/layers/pointnet2.py:43-58 and :114-133, torkit3d/models/classification/pointnet2.py:73-74).

Indices, gathered values and centred coordinates are compared bit for bit; interpolation outputs
(rel 1e-5 / abs 1e-6) and gradients (rel 1e-5 / abs 2e-5: scatter sums whose order differs on the
GPU) within the tolerances the operator tests use.
"""
import numpy as np
import pytest
import torch

from torkit3d_b200 import _fused, workloads
from torkit3d_b200.layers import (FeatureInterpolator, BallQuery, SetAbstractionGrouper, sample_and_gather,
                                  set_abstraction_group, three_nn_interpolate)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def N(t):
    return t.detach().cpu().numpy()


def sphere(B, n, seed):
    g = torch.Generator().manual_seed(seed)
    p = torch.randn(B, n, 3, generator=g)
    p = p / p.norm(dim=2, keepdim=True) + 0.01 * torch.randn(B, n, 3, generator=g)
    return p.contiguous()


def group_np(x, index):
    """x [B,C,N], index [B,M,K] (may hold -1) -> [B,C,M,K]; -1 reads as 0."""
    safe = np.where(index < 0, 0, index)
    out = np.stack([x[b][:, safe[b]] for b in range(x.shape[0])])  # [B,C,M,K]
    return np.where((index >= 0)[:, None], out, 0).astype(x.dtype)


def sa_expected(oracle, pts, cen, feat, radius, K, use_xyz):
    """pts [B,N,3], cen [B,M,3], feat [B,C,N] or None -> (out, index)."""
    index = oracle.ball_query(cen, pts, radius, K)
    parts = []
    if feat is not None:
        parts.append(group_np(feat, index))
    if use_xyz:
        gx = group_np(np.ascontiguousarray(pts.transpose(0, 2, 1)), index)
        parts.append((gx - cen.transpose(0, 2, 1)[..., None]).astype(np.float32))
    return np.concatenate(parts, axis=1), index


# ---- FPS + gather ------------------------------------------------------------------------------
@pytest.mark.parametrize("n,s,dtype", [(1000, 100, torch.float32), (8192, 512, torch.float32),
                                       (9000, 64, torch.float32), (16384, 300, torch.float32), (16500, 40, torch.float32),
                                       (700, 50, torch.float64)])
@pytest.mark.parametrize("channel_first", [True, False])
def test_fps_gather(oracle, n, s, dtype, channel_first):
    p = sphere(3, n, 11).to(dtype)
    want = oracle.fps(p.numpy(), s)
    src = p.transpose(1, 2).contiguous() if channel_first else p
    index, sampled = _fused.fps_gather(src.to(DEV), s, channel_first=channel_first)
    np.testing.assert_array_equal(N(index), want)
    exp = np.take_along_axis(p.numpy(), want[..., None].repeat(3, 2), axis=1)  # [B,S,3]
    got = N(sampled).transpose(0, 2, 1) if channel_first else N(sampled)
    np.testing.assert_array_equal(got, exp)


def test_sample_and_gather_grad():
    p = sphere(2, 600, 12).transpose(1, 2).contiguous().to(DEV).requires_grad_(True)
    index, xyz = sample_and_gather(p, 40)
    w = torch.randn_like(xyz)
    (xyz * w).sum().backward()
    ref = torch.zeros_like(p)
    ref.scatter_add_(2, index.unsqueeze(1).expand(-1, 3, -1), w)
    torch.testing.assert_close(p.grad, ref)


# ---- set-abstraction grouping -------------------------------------------------------------------
SA_CASES = [
    # B, N,   M,   C,  K,  radius, use_xyz
    (2, 2048, 256, 64, 32, 0.2, True),     # vector path
    (2, 2048, 250, 64, 32, 0.2, True),     # ragged last block of centres
    (3, 1000, 100, 6, 10, 0.25, True),     # scalar path (C, K not multiples of 4)
    (2, 1500, 128, 0, 16, 0.2, True),      # coordinates only
    (2, 1500, 128, 32, 16, 0.2, False),    # features only
    (1, 100, 40, 16, 64, 0.5, True),       # cloud smaller than one tile; rows padded
    (2, 3000, 96, 128, 64, 0.15, True),    # wide rows
    (1, 777, 33, 20, 128, 1.0, True),      # K = 128, most of the cloud inside the ball
]


@pytest.mark.parametrize("B,n,M,C,K,radius,use_xyz", SA_CASES)
@pytest.mark.parametrize("channel_first", [True, False])
def test_sa_group_forward(oracle, B, n, M, C, K, radius, use_xyz, channel_first):
    pts = sphere(B, n, 21)
    cen = pts[:, torch.randperm(n, generator=torch.Generator().manual_seed(5))[:M]].contiguous()
    feat = torch.randn(B, C, n, generator=torch.Generator().manual_seed(6)) if C else None
    exp, index = sa_expected(oracle, pts.numpy(), cen.numpy(), feat.numpy() if C else None, radius, K, use_xyz)
    a = pts.transpose(1, 2).contiguous() if channel_first else pts
    c = cen.transpose(1, 2).contiguous() if channel_first else cen
    out, index32 = _fused.sa_group_forward(a.to(DEV), c.to(DEV), feat.to(DEV) if C else None, radius, K,
                                           use_xyz=use_xyz, channel_first=channel_first)
    np.testing.assert_array_equal(N(index32).astype(np.int64), index)
    np.testing.assert_array_equal(N(out), exp)


def test_sa_group_centre_without_neighbour(oracle):
    """A centre far from every point: K entries -1, zero features, coordinates = -centre."""
    pts = sphere(1, 500, 31)
    cen = pts[:, :64].clone()
    cen[0, 7] = torch.tensor([5.0, 5.0, 5.0])
    feat = torch.randn(1, 8, 500, generator=torch.Generator().manual_seed(1))
    exp, index = sa_expected(oracle, pts.numpy(), cen.numpy(), feat.numpy(), 0.2, 16, True)
    assert (index[0, 7] == -1).all()
    out, index32 = _fused.sa_group_forward(pts.to(DEV), cen.to(DEV), feat.to(DEV), 0.2, 16, channel_first=False)
    np.testing.assert_array_equal(N(index32).astype(np.int64), index)
    np.testing.assert_array_equal(N(out), exp)


@pytest.mark.parametrize("C,K", [(64, 32), (6, 10)])
def test_sa_group_backward(oracle, C, K):
    B, n, M = 2, 1500, 200
    pts = sphere(B, n, 41)
    cen = pts[:, :M].contiguous()
    feat = torch.randn(B, C, n, generator=torch.Generator().manual_seed(2))
    a = pts.transpose(1, 2).contiguous().to(DEV).requires_grad_(True)
    c = cen.transpose(1, 2).contiguous().to(DEV).requires_grad_(True)
    f = feat.to(DEV).requires_grad_(True)
    out = set_abstraction_group(a, c, f, 0.2, K, use_xyz=True)
    g = torch.randn(out.shape, generator=torch.Generator().manual_seed(3))
    out.backward(g.to(DEV))
    index = oracle.ball_query(cen.numpy(), pts.numpy(), 0.2, K)
    g64 = g.numpy().astype(np.float64)
    gf = oracle.group_bwd(np.ascontiguousarray(g64[:, :C]), index, n)
    gx = oracle.group_bwd(np.ascontiguousarray(g64[:, C:]), index, n)
    gc = -g64[:, C:].sum(axis=3)
    # sums of up to a few hundred N(0,1) terms in fp32, in a different order: abs error ~ 2^-24 * sum|g|
    np.testing.assert_allclose(N(f.grad), gf, rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(N(a.grad), gx, rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(N(c.grad), gc, rtol=1e-5, atol=2e-5)


def test_sa_grouper_module_matches_operator_chain():
    """The fused module against the same chain spelled with the operators, on the GPU."""
    from torkit3d_b200.ops import ball_query, group_points

    B, n, M, C, K = 2, 4096, 512, 64, 32
    pts = sphere(B, n, 51).transpose(1, 2).contiguous().to(DEV)
    _, cen = sample_and_gather(pts, M)
    feat = torch.randn(B, C, n, device=DEV)
    mod = SetAbstractionGrouper(BallQuery(0.2, K), use_xyz=True)
    out = mod(pts, cen, feat)
    idx = ball_query(cen, pts, 0.2, K)
    ref = torch.cat([group_points(feat, idx), group_points(pts, idx) - cen.unsqueeze(-1)], dim=1)
    assert torch.equal(out, ref)


def test_sa_group_full_c3(oracle):
    """Benchmark configuration (B=32, 8192 points, 1024 centres, r=0.1, K=32, C=64): a slab of
    clouds against the oracle, the whole batch against the operator chain on the GPU."""
    from torkit3d_b200.ops import ball_query, group_points

    p, feat = workloads.c3_set_abstraction()
    pts = p.transpose(1, 2).contiguous().to(DEV)
    _, cen = sample_and_gather(pts, 1024)
    f = feat.to(DEV)
    out = set_abstraction_group(pts, cen, f, 0.1, 32)
    idx = ball_query(cen, pts, 0.1, 32)
    ref = torch.cat([group_points(f, idx), group_points(pts, idx) - cen.unsqueeze(-1)], dim=1)
    assert torch.equal(out, ref)
    sl = slice(0, 2)
    cen_np = N(cen).transpose(0, 2, 1)[sl]
    exp, _ = sa_expected(oracle, p.numpy()[sl], np.ascontiguousarray(cen_np), feat.numpy()[sl], 0.1, 32, True)
    np.testing.assert_array_equal(N(out)[sl], exp)


# ---- three-NN interpolation ----------------------------------------------------------------------
def weights_np(d, eps):
    inv = (np.float32(1.0) / np.maximum(d, np.float32(eps))).astype(np.float32)
    s = ((inv[..., 0] + inv[..., 1]).astype(np.float32) + inv[..., 2]).astype(np.float32)
    return (inv / s[..., None]).astype(np.float32)


# (1, 260000, 1500, 4): about one full round of 256-query blocks per SM; (2, 60000, 900, 4): less than
# one round, where two lanes share a query
@pytest.mark.parametrize("B,nq,nk,C", [(2, 1000, 300, 64), (2, 1001, 257, 6), (1, 4096, 1024, 256), (3, 50, 3, 16),
                                       (1, 260000, 1500, 4), (2, 60000, 900, 4)])
@pytest.mark.parametrize("channel_first", [True, False])
def test_three_nn_interp_forward(oracle, B, nq, nk, C, channel_first):
    g = torch.Generator().manual_seed(61)
    q = torch.rand(B, nq, 3, generator=g)
    k = torch.rand(B, nk, 3, generator=g)
    k[:, 0] = q[:, 0]  # an exact hit: distance 0 is clamped to eps
    feat = torch.randn(B, C, nk, generator=g)
    d, idx = oracle.knn(q.numpy(), k.numpy(), 3)
    w = weights_np(d, 1e-10)
    exp = oracle.interp_fwd(feat.numpy().astype(np.float64), idx, w.astype(np.float64))
    qq = q.transpose(1, 2).contiguous() if channel_first else q
    kk = k.transpose(1, 2).contiguous() if channel_first else k
    out, index32, weight = _fused.three_nn_interp_forward(qq.to(DEV), kk.to(DEV), feat.to(DEV), eps=1e-10,
                                                          channel_first=channel_first)
    np.testing.assert_array_equal(N(index32).astype(np.int64), idx)
    np.testing.assert_allclose(N(weight), w, rtol=1e-6, atol=0)
    np.testing.assert_allclose(N(out), exp, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("nq,C", [(1000, 64), (1001, 6)])
def test_three_nn_interp_backward(oracle, nq, C):
    B, nk = 2, 300
    g = torch.Generator().manual_seed(62)
    q = torch.rand(B, 3, nq, generator=g)
    k = torch.rand(B, 3, nk, generator=g)
    feat = torch.randn(B, C, nk, generator=g)
    f = feat.to(DEV).requires_grad_(True)
    out = FeatureInterpolator()(q.to(DEV), k.to(DEV), f)
    go = torch.randn(out.shape, generator=g)
    out.backward(go.to(DEV))
    d, idx = oracle.knn(np.ascontiguousarray(q.numpy().transpose(0, 2, 1)),
                        np.ascontiguousarray(k.numpy().transpose(0, 2, 1)), 3)
    w = weights_np(d, 1e-10).astype(np.float64)
    exp = oracle.interp_bwd(go.numpy().astype(np.float64), idx, w, nk)
    np.testing.assert_allclose(N(f.grad), exp, rtol=1e-5, atol=2e-5)


def test_three_nn_interpolate_matches_operator_chain():
    from torkit3d_b200.ops import interpolate_feature, knn_points

    g = torch.Generator().manual_seed(63)
    q = (torch.rand(2, 3, 5000, generator=g) * 5).to(DEV)
    k = (torch.rand(2, 3, 1200, generator=g) * 5).to(DEV)
    feat = torch.randn(2, 128, 1200, generator=g).to(DEV)
    out = three_nn_interpolate(q, k, feat)
    d, idx = knn_points(q, k, 3, transpose=True)
    inv = 1.0 / torch.clamp(d, min=1e-10)
    w = inv / inv.sum(dim=2, keepdim=True)
    ref = interpolate_feature(feat, idx, w)
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-6)


def test_fused_rejects_unsupported():
    pts = sphere(1, 64, 71).to(DEV)
    with pytest.raises(RuntimeError):
        _fused.sa_group_forward(pts, pts[:, :8].contiguous(), None, 0.2, 129, channel_first=False)  # K > 128
    with pytest.raises(RuntimeError):
        _fused.three_nn_interp_forward(pts, pts[:, :2].contiguous(), torch.zeros(1, 4, 2, device=DEV),
                                       channel_first=False)  # fewer than 3 keys


# ---- EdgeConv edge features -----------------------------------------------------------------------
def edge_expected(q, k, index, include_query):
    grouped = group_np(k, index)
    qe = np.broadcast_to(q[..., None], grouped.shape)
    edge = (grouped - qe).astype(q.dtype)
    return np.concatenate([edge, qe], axis=1) if include_query else edge


@pytest.mark.parametrize("B,C,n1,n2,K,dtype", [
    (2, 64, 1024, 1024, 20, torch.float32),   # row path (DGCNN shape)
    (2, 6, 500, 700, 20, torch.float32),      # direct path: C not a multiple of 4
    (1, 128, 333, 400, 7, torch.float32),     # direct path: N1*K not a multiple of 4
    (2, 8, 300, 300, 3, torch.float32),       # K smaller than a 16-byte chunk
    (2, 16, 200, 260, 10, torch.float64),
])
@pytest.mark.parametrize("include_query", [True, False])
def test_edge_feature_forward(B, C, n1, n2, K, dtype, include_query):
    from torkit3d_b200.ops import get_edge_feature

    g = torch.Generator().manual_seed(81)
    q = torch.randn(B, C, n1, generator=g, dtype=dtype)
    k = torch.randn(B, C, n2, generator=g, dtype=dtype)
    index = torch.randint(0, n2, (B, n1, K), generator=g)
    out = get_edge_feature(q.to(DEV), k.to(DEV), index.to(DEV), include_query)
    np.testing.assert_array_equal(N(out), edge_expected(q.numpy(), k.numpy(), index.numpy(), include_query))


@pytest.mark.parametrize("C,n1,K", [(64, 512, 20), (6, 300, 7)])
def test_edge_feature_backward(oracle, C, n1, K):
    from torkit3d_b200.ops import get_edge_feature

    B, n2 = 2, 400
    g = torch.Generator().manual_seed(82)
    q = torch.randn(B, C, n1, generator=g)
    k = torch.randn(B, C, n2, generator=g)
    index = torch.randint(0, n2, (B, n1, K), generator=g)
    qd, kd = q.to(DEV).requires_grad_(True), k.to(DEV).requires_grad_(True)
    out = get_edge_feature(qd, kd, index.to(DEV))
    go = torch.randn(out.shape, generator=g)
    out.backward(go.to(DEV))
    g64 = go.numpy().astype(np.float64)
    gk = oracle.group_bwd(np.ascontiguousarray(g64[:, :C]), index.numpy(), n2)
    gq = (g64[:, C:] - g64[:, :C]).sum(axis=3)
    np.testing.assert_allclose(N(kd.grad), gk, rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(N(qd.grad), gq, rtol=1e-5, atol=2e-5)


def test_edge_feature_matches_operator_chain():
    from torkit3d_b200.ops import get_edge_feature, group_points, knn_points

    B, C, n, K = 4, 64, 2048, 20
    pts = sphere(B, n, 83).to(DEV)
    _, ind = knn_points(pts, pts, K)
    x = torch.randn(B, C, n, device=DEV)
    out = get_edge_feature(x, x, ind)
    grouped = group_points(x, ind)
    ref = torch.cat([grouped - x.unsqueeze(3), x.unsqueeze(3).expand_as(grouped)], dim=1)
    assert torch.equal(out, ref)


# ---- golden fixtures produced by the reference's own layer code (tests/golden/make_golden.py) ---------
def test_golden_fps_gather(golden):
    g = golden("fps_gather")
    for tag in "ab":
        idx, xyz = sample_and_gather(torch.from_numpy(g[tag + "_points"]).to(DEV), int(g[tag + "_s"]))
        np.testing.assert_array_equal(N(idx), g[tag + "_index"])
        np.testing.assert_array_equal(N(xyz), g[tag + "_xyz"])


def test_golden_sa_group(golden):
    g = golden("sa_group")
    for tag in "abcd":
        feat = torch.from_numpy(g[tag + "_feature"]).to(DEV) if (tag + "_feature") in g.files else None
        out = set_abstraction_group(torch.from_numpy(g[tag + "_in_xyz"]).to(DEV),
                                    torch.from_numpy(g[tag + "_out_xyz"]).to(DEV), feat, float(g[tag + "_radius"]),
                                    int(g[tag + "_k"]), bool(g[tag + "_use_xyz"]))
        np.testing.assert_array_equal(N(out), g[tag + "_nbr"])


def test_golden_edge_feature(golden):
    from torkit3d_b200.ops import get_edge_feature

    g = golden("edge_feature")
    for tag in "ab":
        q, k, i = [torch.from_numpy(g[tag + n]).to(DEV) for n in ("_query", "_key", "_index")]
        np.testing.assert_array_equal(N(get_edge_feature(q, k, i)), g[tag + "_edge"])
        np.testing.assert_array_equal(N(get_edge_feature(q, k, i, include_query=False)), g[tag + "_edge_noquery"])


def test_golden_three_nn_interp(golden):
    g = golden("three_nn_interp")
    for tag in "ab":
        q, k, f = [torch.from_numpy(g[tag + n]).to(DEV) for n in ("_query", "_key", "_feature")]
        out = FeatureInterpolator()(q, k, f)
        # the reference formulation gets its distances from cdist (a square root, squared again)
        np.testing.assert_allclose(N(out), g[tag + "_out"], rtol=1e-4, atol=1e-5)
