"""The CPU oracle against the fixtures produced by the reference's own Python formulations
(tests/golden/make_golden.py), and against the restated formulations on fresh inputs."""
import numpy as np
import pytest
import torch

from oracle import formulations as F


def test_chamfer_golden(oracle, golden):
    g = golden("chamfer")
    for tag in ("f32", "f64"):
        d1, i1, d2, i2 = oracle.chamfer_fwd(g[tag + "_xyz1"], g[tag + "_xyz2"])
        # torch's sum over the last axis of diff**2 is the un-fused (x^2+y^2)+z^2: bit-exact.
        np.testing.assert_array_equal(i1, g[tag + "_idx1"])
        np.testing.assert_array_equal(i2, g[tag + "_idx2"])
        np.testing.assert_array_equal(d1, g[tag + "_dist1"])
        np.testing.assert_array_equal(d2, g[tag + "_dist2"])
        B, N = d1.shape
        M = d2.shape[1]
        g1 = np.full((B, N), 1.0 / (B * N), d1.dtype)
        g2 = np.full((B, M), 1.0 / (B * M), d1.dtype)
        ga, gb = oracle.chamfer_bwd(g1, g2, g[tag + "_xyz1"], g[tag + "_xyz2"], i1, i2)
        tol = dict(rtol=1e-5, atol=1e-6) if tag == "f32" else dict(rtol=1e-10, atol=1e-12)
        np.testing.assert_allclose(ga, g[tag + "_grad1"], **tol)
        np.testing.assert_allclose(gb, g[tag + "_grad2"], **tol)


def test_knn_golden(oracle, golden):
    g = golden("knn")
    for tag in "abc":
        k = int(g[tag + "_k"])
        d, i = oracle.knn(g[tag + "_query"], g[tag + "_key"], k)
        np.testing.assert_array_equal(i, g[tag + "_idx"])
        # the reference formulation returns Euclidean distances through cdist
        np.testing.assert_allclose(np.sqrt(d), g[tag + "_dist"], rtol=1e-4, atol=5e-5)


def test_feature_knn_golden(oracle, golden):
    """The reference's native.knn (cdist + topk) on float64 features: same neighbours, same distances.
    The float32 oracle (the arithmetic the CUDA kernel follows) agrees with it up to rounding."""
    g = golden("feature_knn")
    for tag in "abcd":
        k, cf = int(g[tag + "_k"]), bool(g[tag + "_cf"])
        q, r = g[tag + "_query"], g[tag + "_key"]
        d, i = oracle.feature_knn(q, r, k, channel_first=cf)
        np.testing.assert_array_equal(i, g[tag + "_idx"])
        np.testing.assert_allclose(np.sqrt(d), g[tag + "_dist"], rtol=1e-9, atol=1e-9)
        d32, i32 = oracle.feature_knn(q.astype(np.float32), r.astype(np.float32), k, channel_first=cf)
        assert (i32 == g[tag + "_idx"]).mean() > 0.995
        np.testing.assert_allclose(np.sqrt(d32), g[tag + "_dist"], rtol=1e-5, atol=1e-6)


def test_fps_golden(oracle, golden):
    g = golden("fps")
    for tag in "abcd":
        idx = oracle.fps(g[tag + "_points"], int(g[tag + "_s"]))
        np.testing.assert_array_equal(idx, g[tag + "_idx"])


def test_ball_query_golden(oracle, golden):
    g = golden("ball_query")
    for tag in "abcd":
        idx = oracle.ball_query(g[tag + "_query"], g[tag + "_key"], float(g[tag + "_r"]), int(g[tag + "_k"]))
        np.testing.assert_array_equal(idx, g[tag + "_idx"])


def test_group_golden(oracle, golden):
    g = golden("group_points")
    for tag in "ab":
        out = oracle.group_fwd(g[tag + "_feature"], g[tag + "_index"])
        np.testing.assert_array_equal(out, g[tag + "_out"])
        gin = oracle.group_bwd(np.ones_like(out), g[tag + "_index"], g[tag + "_feature"].shape[2])
        np.testing.assert_allclose(gin, g[tag + "_grad"], rtol=1e-6, atol=1e-6)


def test_interpolate_golden(oracle, golden):
    g = golden("interpolate")
    for tag in "ab":
        out = oracle.interp_fwd(g[tag + "_feature"], g[tag + "_index"], g[tag + "_weight"])
        np.testing.assert_allclose(out, g[tag + "_out"], rtol=1e-12, atol=1e-14)
        gin = oracle.interp_bwd(np.ones_like(out), g[tag + "_index"], g[tag + "_weight"], g[tag + "_feature"].shape[2])
        np.testing.assert_allclose(gin, g[tag + "_grad"], rtol=1e-10, atol=1e-12)


# ---- oracle vs the restated formulations on fresh inputs, fp32, including exact ties ----------

def _tie_cloud(rng, B, N):
    """Points on a coarse grid with duplicates: many exactly equal distances."""
    p = rng.integers(-3, 4, size=(B, N, 3)).astype(np.float32) * 0.25
    return p


@pytest.mark.parametrize("ties", [False, True])
def test_chamfer_vs_formulation(oracle, ties):
    rng = np.random.default_rng(5)
    a = _tie_cloud(rng, 3, 257) if ties else rng.standard_normal((3, 257, 3)).astype(np.float32)
    b = _tie_cloud(rng, 3, 130) if ties else rng.standard_normal((3, 130, 3)).astype(np.float32)
    d1, i1, d2, i2 = oracle.chamfer_fwd(a, b)
    e1, j1, e2, j2 = F.chamfer_dense(torch.from_numpy(a), torch.from_numpy(b))
    np.testing.assert_array_equal(d1, e1.numpy())
    np.testing.assert_array_equal(d2, e2.numpy())
    if not ties:  # torch.min does not promise the first index among equal minima
        np.testing.assert_array_equal(i1, j1.numpy())
        np.testing.assert_array_equal(i2, j2.numpy())
    else:
        full = F.pairwise_sqdist(torch.from_numpy(a), torch.from_numpy(b)).numpy()
        np.testing.assert_array_equal(i1, full.argmin(2))  # numpy argmin: first minimum
        np.testing.assert_array_equal(i2, full.argmin(1))


@pytest.mark.parametrize("ties", [False, True])
def test_knn_vs_formulation(oracle, ties):
    rng = np.random.default_rng(6)
    q = _tie_cloud(rng, 2, 100) if ties else rng.standard_normal((2, 100, 3)).astype(np.float32)
    r = _tie_cloud(rng, 2, 333) if ties else rng.standard_normal((2, 333, 3)).astype(np.float32)
    k = 16
    d, i = oracle.knn(q, r, k)
    full = F.pairwise_sqdist(torch.from_numpy(q), torch.from_numpy(r)).numpy()
    order = np.argsort(full, axis=2, kind="stable")[:, :, :k]  # stable: ties keep the lower index first
    np.testing.assert_array_equal(i, order)
    np.testing.assert_array_equal(d, np.take_along_axis(full, order, 2))


def test_fps_vs_formulation(oracle):
    rng = np.random.default_rng(7)
    p = rng.random((3, 500, 3)).astype(np.float32)
    np.testing.assert_array_equal(oracle.fps(p, 64), F.fps_numpy(p, 64))
    # duplicated points: exact ties for the maximum go to the lowest index (numpy argmax)
    p = np.concatenate([p[:, :250], p[:, :250]], axis=1)
    np.testing.assert_array_equal(oracle.fps(p, 300), F.fps_numpy(p, 300))


def test_ball_query_vs_formulation(oracle):
    rng = np.random.default_rng(8)
    key = rng.standard_normal((2, 200, 3)).astype(np.float32)
    query = rng.standard_normal((2, 50, 3)).astype(np.float32) * 2  # some rows have no hit at all
    r = np.float32(0.3)
    got = oracle.ball_query(query, key, float(r), 8)
    np.testing.assert_array_equal(got, F.ball_query_numpy(query, key, r, 8))
    assert (got == -1).any() and (got >= 0).any()


def test_three_nn_weight_vs_formulation(oracle):
    rng = np.random.default_rng(9)
    d = rng.random((4, 50, 3)).astype(np.float32)
    d[0, 0, 0] = 0.0
    w = oracle.three_nn_weight(d)
    np.testing.assert_allclose(w, F.three_nn_weight(torch.from_numpy(d)).numpy(), rtol=1e-6)
    np.testing.assert_allclose(w.sum(-1), 1.0, rtol=1e-5)


def test_empty_and_edge(oracle):
    a = np.zeros((2, 5, 3), np.float32)
    b = np.zeros((2, 0, 3), np.float32)
    d1, i1, d2, i2 = oracle.chamfer_fwd(a, b)
    assert np.isinf(d1).all() and (i1 == -1).all() and d2.shape == (2, 0)
    # all points identical: FPS keeps returning index 0 (argmax of an all-zero array)
    p = np.ones((1, 10, 3), np.float32)
    assert (oracle.fps(p, 5) == 0).all()
    # k == N2
    q = np.random.default_rng(1).standard_normal((1, 4, 3)).astype(np.float32)
    d, i = oracle.knn(q, q, 4)
    assert (np.sort(i, 2) == np.arange(4)).all() and (i[:, :, 0] == np.arange(4)).all()


# ---- callers of the operators: the oracle's compositions against the reference's own layer code ----
def test_fps_gather_golden(oracle, golden):
    g = golden("fps_gather")
    for tag in "ab":
        idx, xyz = oracle.fps_gather(g[tag + "_points"], int(g[tag + "_s"]))
        np.testing.assert_array_equal(idx, g[tag + "_index"])
        np.testing.assert_array_equal(xyz, g[tag + "_xyz"])


def test_sa_group_golden(oracle, golden):
    g = golden("sa_group")
    for tag in "abcd":
        feat = g[tag + "_feature"] if (tag + "_feature") in g.files else None
        out, _ = oracle.sa_group(g[tag + "_in_xyz"], g[tag + "_out_xyz"], feat, float(g[tag + "_radius"]),
                                 int(g[tag + "_k"]), bool(g[tag + "_use_xyz"]))
        np.testing.assert_array_equal(out, g[tag + "_nbr"])


def test_edge_feature_golden(oracle, golden):
    g = golden("edge_feature")
    for tag in "ab":
        np.testing.assert_array_equal(oracle.edge_feature(g[tag + "_query"], g[tag + "_key"], g[tag + "_index"]),
                                      g[tag + "_edge"])
        np.testing.assert_array_equal(
            oracle.edge_feature(g[tag + "_query"], g[tag + "_key"], g[tag + "_index"], include_query=False),
            g[tag + "_edge_noquery"])


def test_three_nn_interp_golden(oracle, golden):
    g = golden("three_nn_interp")
    for tag in "ab":
        out, _, _ = oracle.three_nn_interp(g[tag + "_query"], g[tag + "_key"], g[tag + "_feature"])
        # the reference formulation gets its distances from cdist (a square root, squared again)
        np.testing.assert_allclose(out, g[tag + "_out"], rtol=1e-4, atol=1e-5)
