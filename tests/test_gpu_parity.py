"""GPU parity: the CUDA library (through the operator layer and the C ABI) against the CPU oracle
and the golden fixtures.  Indices and forward distances must be bit-exact; gradients and
interpolated features within rel 1e-5 / abs 1e-6 (fp32)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
GRAD_TOL = dict(rtol=1e-5, atol=1e-6)


def T(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV)


def N(t):
    return t.detach().cpu().numpy()


def grid_cloud(rng, B, n, dtype=np.float32):
    """Coarse grid with duplicates: many exactly tied distances."""
    return (rng.integers(-3, 4, size=(B, n, 3)) * 0.25).astype(dtype)


# ------------------------------------------------------------------------------------------- chamfer
CHAMFER_SHAPES = [(1, 1, 1), (2, 31, 33), (3, 127, 129), (2, 128, 512), (1, 513, 1000), (2, 1024, 1024),
                  (5, 700, 64), (64, 600, 601), (8, 2100, 2050)]


@pytest.mark.parametrize("B,n1,n2", CHAMFER_SHAPES)
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_chamfer_forward_bit_exact(oracle, B, n1, n2, dtype):
    from torkit3d_b200.ops import nn_distance

    if dtype == np.float64 and B * n1 * n2 > 5_000_000:
        pytest.skip("fp64 generic path covered by the smaller shapes")
    rng = np.random.default_rng(B * 1000 + n1)
    a = rng.standard_normal((B, n1, 3)).astype(dtype)
    b = rng.standard_normal((B, n2, 3)).astype(dtype)
    d1, i1, d2, i2 = [N(t) for t in nn_distance(T(a), T(b))]
    e1, j1, e2, j2 = oracle.chamfer_fwd(a, b)
    np.testing.assert_array_equal(i1, j1)
    np.testing.assert_array_equal(i2, j2)
    np.testing.assert_array_equal(d1, e1)
    np.testing.assert_array_equal(d2, e2)


# Few queries: 2, 4 or 8 lanes share a query; clouds of very different sizes: one launch per
# direction, each with its own shape.  Lattice clouds give exact ties across the lanes' key groups.
@pytest.mark.parametrize("B,n1,n2", [(2, 1024, 1024), (4, 4096, 4096), (6, 1000, 3000), (1, 300, 50000), (2, 30000, 777),
                                     (1, 17, 9000), (3, 9000, 2), (2, 70000, 1000), (1, 8192, 8192)])
@pytest.mark.parametrize("lattice", [False, True])
def test_chamfer_forward_few_queries_and_unequal_clouds(oracle, B, n1, n2, lattice):
    from torkit3d_b200.ops import nn_distance

    rng = np.random.default_rng(B * 77 + n1 + n2)
    if lattice:
        a = (rng.integers(-12, 13, size=(B, n1, 3)) / 4).astype(np.float32)
        b = (rng.integers(-12, 13, size=(B, n2, 3)) / 4).astype(np.float32)
    else:
        a = rng.standard_normal((B, n1, 3)).astype(np.float32)
        b = rng.standard_normal((B, n2, 3)).astype(np.float32)
    d1, i1, d2, i2 = [N(t) for t in nn_distance(T(a), T(b))]
    e1, j1, e2, j2 = oracle.chamfer_fwd(a, b)
    np.testing.assert_array_equal(i1, j1)
    np.testing.assert_array_equal(i2, j2)
    np.testing.assert_array_equal(d1, e1)
    np.testing.assert_array_equal(d2, e2)


# At least 148 * 512 queries but no more than two rounds of 256-query tasks per SM: the launcher
# runs these as one 896-thread block per SM (seven independent 128-thread groups).
SM_WIDE_SHAPES = [(3, 20001, 9999), (1, 100000, 3), (2, 70000, 0), (8, 16384, 16384), (16, 4097, 5003),
                  (5, 16000, 30000)]


@pytest.mark.parametrize("B,n1,n2", SM_WIDE_SHAPES)
def test_chamfer_forward_sm_wide_path_bit_exact(oracle, B, n1, n2):
    from torkit3d_b200 import _C

    rng = np.random.default_rng(B * 7 + n2)
    if B == 8:   # one rank's share of the 8-GPU benchmark batch, checked on two of its clouds
        from torkit3d_b200 import workloads
        a, b = [t.numpy() for t in workloads.c4_chamfer_large(B=8)]
        check = [2, 7]
    else:        # coarse lattice: plenty of exactly tied distances
        a = (rng.integers(-40, 41, size=(B, n1, 3)) / 16).astype(np.float32)
        b = (rng.integers(-40, 41, size=(B, n2, 3)) / 16).astype(np.float32)
        check = list(range(B))
    sums = torch.zeros(2, dtype=torch.float64, device="cuda")
    d1, i1, d2, i2 = [N(t) for t in _C.chamfer_distance_forward_cuda(T(a), T(b), sums=sums)]
    e1, j1, e2, j2 = oracle.chamfer_fwd(a[check], b[check])
    np.testing.assert_array_equal(i1[check], j1)
    np.testing.assert_array_equal(i2[check], j2)
    np.testing.assert_array_equal(d1[check], e1)
    np.testing.assert_array_equal(d2[check], e2)
    if n2 > 0:
        np.testing.assert_allclose(N(sums), [d1.sum(dtype=np.float64), d2.sum(dtype=np.float64)], rtol=1e-12)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_chamfer_ties_go_to_lowest_index(oracle, dtype):
    from torkit3d_b200.ops import nn_distance

    rng = np.random.default_rng(3)
    a, b = grid_cloud(rng, 4, 777, dtype), grid_cloud(rng, 4, 1500, dtype)
    d1, i1, d2, i2 = [N(t) for t in nn_distance(T(a), T(b))]
    e1, j1, e2, j2 = oracle.chamfer_fwd(a, b)
    np.testing.assert_array_equal(i1, j1)
    np.testing.assert_array_equal(i2, j2)
    np.testing.assert_array_equal(d1, e1)


def test_chamfer_far_from_origin_and_huge_values(oracle):
    """The fp32 filter must stay conservative where its cheap estimate is useless."""
    from torkit3d_b200.ops import nn_distance

    rng = np.random.default_rng(4)
    # last case: |p|^2 overflows fp32 for every point while all distances are finite
    for offset, scale in ((1000.0, 1.0), (-3.0e4, 10.0), (0.0, 1e-20), (0.0, 1e18), (5e18, 1e18), (1.85e19, 1e17)):
        a = (rng.standard_normal((2, 300, 3)) * scale + offset).astype(np.float32)
        b = (rng.standard_normal((2, 700, 3)) * scale + offset).astype(np.float32)
        d1, i1, d2, i2 = [N(t) for t in nn_distance(T(a), T(b))]
        e1, j1, e2, j2 = oracle.chamfer_fwd(a, b)
        np.testing.assert_array_equal(i1, j1)
        np.testing.assert_array_equal(i2, j2)
        np.testing.assert_array_equal(d1, e1)
        np.testing.assert_array_equal(d2, e2)


def test_knn_and_ball_query_where_squared_norms_overflow(oracle):
    """Coordinates near 1.85e19: |p|^2 = inf in fp32, pairwise distances about 1e34."""
    from torkit3d_b200.ops import ball_query, knn_points

    rng = np.random.default_rng(5)
    q = (rng.standard_normal((2, 200, 3)) * 1e17 + 1.85e19).astype(np.float32)
    r = (rng.standard_normal((2, 600, 3)) * 1e17 + 1.85e19).astype(np.float32)
    for k in (3, 16):
        d, i = knn_points(T(q), T(r), k)
        ed, ei = oracle.knn(q, r, k)
        np.testing.assert_array_equal(N(i), ei)
        np.testing.assert_array_equal(N(d), ed)
    idx = ball_query(T(q), T(r), 1.5e17, 8, transpose=False)
    np.testing.assert_array_equal(N(idx), oracle.ball_query(q, r, 1.5e17, 8))


def test_chamfer_empty_partner_and_empty_batch():
    from torkit3d_b200.ops import nn_distance

    a = torch.randn(2, 5, 3, device=DEV)
    b = torch.zeros(2, 0, 3, device=DEV)
    d1, i1, d2, i2 = nn_distance(a, b)
    assert torch.isinf(d1).all() and (i1 == -1).all() and d2.shape == (2, 0) and i2.shape == (2, 0)
    d1, i1, d2, i2 = nn_distance(torch.zeros(0, 5, 3, device=DEV), torch.zeros(0, 7, 3, device=DEV))
    assert d1.shape == (0, 5) and d2.shape == (0, 7)


def test_chamfer_golden_and_layouts(golden):
    from torkit3d_b200.ops import chamfer_distance

    g = golden("chamfer")
    for tag in ("f32", "f64"):
        x1 = T(g[tag + "_xyz1"]).requires_grad_(True)
        x2 = T(g[tag + "_xyz2"]).requires_grad_(True)
        d1, d2 = chamfer_distance(x1, x2)
        np.testing.assert_array_equal(N(d1), g[tag + "_dist1"])
        np.testing.assert_array_equal(N(d2), g[tag + "_dist2"])
        (d1.mean() + d2.mean()).backward()
        tol = GRAD_TOL if tag == "f32" else dict(rtol=1e-10, atol=1e-12)
        np.testing.assert_allclose(N(x1.grad), g[tag + "_grad1"], **tol)
        np.testing.assert_allclose(N(x2.grad), g[tag + "_grad2"], **tol)
        # channel-first inputs and the 2-D (unbatched) form
        t1, t2 = chamfer_distance(x1.detach().transpose(1, 2), x2.detach().transpose(1, 2), transpose=True)
        assert torch.equal(t1, d1) and torch.equal(t2, d2)
        u1, u2 = chamfer_distance(x1.detach()[0], x2.detach()[0])
        assert torch.equal(u1[0], d1[0]) and torch.equal(u2[0], d2[0])
        s1, _ = chamfer_distance(x1.detach(), x2.detach(), sqrt=True)
        np.testing.assert_allclose(N(s1), np.sqrt(np.maximum(g[tag + "_dist1"], 1e-12)), rtol=1e-6)


@pytest.mark.parametrize("B,n1,n2", [(2, 100, 130), (3, 1024, 1024), (2, 3000, 500)])
def test_chamfer_backward_vs_oracle(oracle, B, n1, n2):
    from torkit3d_b200 import _C

    rng = np.random.default_rng(11)
    a = rng.standard_normal((B, n1, 3)).astype(np.float32)
    b = rng.standard_normal((B, n2, 3)).astype(np.float32)
    g1 = rng.standard_normal((B, n1)).astype(np.float32)
    g2 = rng.standard_normal((B, n2)).astype(np.float32)
    _, i1, _, i2 = oracle.chamfer_fwd(a, b)
    ga, gb = _C.chamfer_distance_backward_cuda(T(g1), T(g2), T(a), T(b), T(i1), T(i2))
    ea, eb = oracle.chamfer_bwd(g1.astype(np.float64), g2.astype(np.float64), a.astype(np.float64),
                                b.astype(np.float64), i1, i2)
    np.testing.assert_allclose(N(ga), ea, rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(N(gb), eb, rtol=1e-5, atol=2e-6)


def test_chamfer_gradcheck_fp64():
    from torkit3d_b200.ops import chamfer_distance

    torch.manual_seed(0)
    x1 = torch.rand(2, 64, 3, dtype=torch.float64, device=DEV, requires_grad=True)
    x2 = torch.rand(2, 50, 3, dtype=torch.float64, device=DEV, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a, b: chamfer_distance(a, b), (x1, x2), eps=1e-6, atol=1e-4,
                                    nondet_tol=1e-9)


def test_chamfer_partial_sums():
    from torkit3d_b200 import _C

    a = torch.randn(7, 1500, 3, device=DEV)
    b = torch.randn(7, 900, 3, device=DEV)
    sums = torch.full((2,), 123.0, dtype=torch.float64, device=DEV)
    d1, _, d2, _ = _C.chamfer_distance_forward_cuda(a, b, sums=sums)
    np.testing.assert_allclose(N(sums), [N(d1).astype(np.float64).sum(), N(d2).astype(np.float64).sum()], rtol=1e-12)


# ----------------------------------------------------------------------------------------------- knn
KNN_CASES = [(1, 1, 1, 1), (2, 33, 64, 1), (2, 100, 300, 3), (3, 511, 1025, 31), (2, 512, 1024, 32), (1, 700, 2000, 4),
             (2, 257, 900, 5), (4, 1000, 1111, 16), (2, 300, 1300, 64), (1, 200, 700, 100), (1, 130, 400, 128),
             (1, 64, 300, 200), (2, 50, 16, 16), (40, 600, 700, 16), (40, 600, 700, 3),
             # two-pass variants with 64 / 128 / 256 key classes (need N2 >= 32 k)
             (2, 300, 2100, 20), (2, 300, 2100, 32), (2, 257, 2200, 64), (1, 100, 3300, 65), (1, 200, 4200, 100),
             (1, 130, 4100, 128),
             # radix selection: k > 80, or k > 40 on small key clouds; k up to 256, N2 == k
             (2, 70, 5000, 81), (2, 300, 300, 64), (2, 100, 256, 256), (3, 65, 1500, 256), (1, 33, 700, 41),
             (1, 40, 20000, 150)]


@pytest.mark.parametrize("B,n1,n2,k", KNN_CASES)
def test_knn_bit_exact(oracle, B, n1, n2, k):
    from torkit3d_b200.ops import knn_points

    rng = np.random.default_rng(n1 * 7 + k)
    q = rng.standard_normal((B, n1, 3)).astype(np.float32)
    r = rng.standard_normal((B, n2, 3)).astype(np.float32)
    d, i = knn_points(T(q), T(r), k)
    e, j = oracle.knn(q, r, k)
    np.testing.assert_array_equal(N(i), j)
    np.testing.assert_array_equal(N(d), e)


@pytest.mark.parametrize("k", [20, 32, 64, 128])
def test_knn_large_k_with_massive_ties(oracle, k):
    """Every key appears 8 times and many queries coincide with keys: candidate lists overflow and
    the exact fallback has to reproduce the (distance, index) order."""
    from torkit3d_b200.ops import knn_points

    rng = np.random.default_rng(k)
    base = rng.standard_normal((2, 520, 3)).astype(np.float32)
    r = np.tile(base, (1, 8, 1))  # 4160 keys
    q = np.concatenate([base[:, :100], rng.standard_normal((2, 100, 3)).astype(np.float32)], axis=1)
    d, i = knn_points(T(q), T(r), k)
    e, j = oracle.knn(q, r, k)
    np.testing.assert_array_equal(N(i), j)
    np.testing.assert_array_equal(N(d), e)


@pytest.mark.parametrize("k", [1, 3, 4, 8, 16, 50, 150, 256])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_knn_ties(oracle, k, dtype):
    from torkit3d_b200.ops import knn_points

    rng = np.random.default_rng(k)
    q, r = grid_cloud(rng, 2, 300, dtype), grid_cloud(rng, 2, 900, dtype)
    d, i = knn_points(T(q), T(r), k, sorted=True)
    e, j = oracle.knn(q, r, k)
    np.testing.assert_array_equal(N(i), j)
    np.testing.assert_array_equal(N(d), e)


@pytest.mark.parametrize("n1,n2,k,dtype", [(300, 500, 3, np.float32),      # register top-k
                                           (300, 1200, 16, np.float32),    # two-pass candidate lists
                                           (300, 2100, 64, np.float32),
                                           (300, 100, 16, np.float32),     # buffered lists
                                           (64, 600, 200, np.float32),     # radix selection
                                           (64, 600, 300, np.float32),     # heap in the output row
                                           (300, 600, 8, np.float64),      # key-split heaps
                                           (64, 400, 100, np.float64)])
def test_knn_keys_with_nan_coordinates_order_last(oracle, n1, n2, k, dtype):
    """A key with a NaN coordinate has a NaN distance to every query; it orders after every number,
    so with at least k numeric keys it is never returned -- also when it is among the first k keys,
    where a set maintained with a plain `<` against its maximum would keep it for good (the
    reference's bounded set does, torkit3d/csrc/include/mink.cuh:70-84)."""
    from torkit3d_b200.ops import knn_points

    rng = np.random.default_rng(n2 + k)
    q = rng.standard_normal((2, n1, 3)).astype(dtype)
    r = rng.standard_normal((2, n2, 3)).astype(dtype)
    bad = rng.random((2, n2)) < 0.1
    bad[:, [0, 2, 5]] = True
    r[bad, rng.integers(0, 3, size=int(bad.sum()))] = np.nan
    d, i = knn_points(T(q), T(r), k, sorted=True)
    e, j = oracle.knn(q, r, k)
    assert not np.isnan(e).any() and not bad[np.arange(2)[:, None, None], j].any()
    np.testing.assert_array_equal(N(i), j)
    np.testing.assert_array_equal(N(d), e)


@pytest.mark.parametrize("k", [1, 2, 3, 4])
@pytest.mark.parametrize("n2", [700, 3001])
def test_knn_small_two_lanes_per_query_bit_exact(oracle, k, n2):
    """Less than one round of 256-query blocks (here 100000 queries: about 2.6 blocks per SM): two
    lanes share a query, sweep alternate key groups and merge their lists; a lattice gives exact
    ties across the two lanes' groups, which must still resolve to the lowest index."""
    from torkit3d_b200.ops import knn_points

    rng = np.random.default_rng(70 + k)
    q = (rng.integers(-30, 31, size=(2, 50000, 3)) / 8).astype(np.float32)
    r = (rng.integers(-30, 31, size=(2, n2, 3)) / 8).astype(np.float32)
    d, i = knn_points(T(q), T(r), k, sorted=True)
    e, j = oracle.knn(q, r, k)
    np.testing.assert_array_equal(N(i), j)
    np.testing.assert_array_equal(N(d), e)
    q2 = rng.standard_normal((1, 90001, 3)).astype(np.float32)
    r2 = rng.standard_normal((1, 1234, 3)).astype(np.float32)
    d, i = knn_points(T(q2), T(r2), k, sorted=True)
    e, j = oracle.knn(q2, r2, k)
    np.testing.assert_array_equal(N(i), j)
    np.testing.assert_array_equal(N(d), e)


@pytest.mark.parametrize("k", [1, 3, 4])
@pytest.mark.parametrize("B,n1,n2", [(2, 20000, 1500), (2, 5000, 2600), (1, 1500, 5000), (1, 77, 9000)])
def test_knn_small_several_lanes_per_query_bit_exact(oracle, k, B, n1, n2):
    """Few queries: 2, 4 or 8 lanes share a query (40000, 10000, 1500 and 77 queries here), sweep
    every 2nd / 4th / 8th key group and merge their lists in butterfly steps; lattice clouds give
    exact ties across the lanes' groups, which must resolve to the lowest index."""
    from torkit3d_b200.ops import knn_points

    rng = np.random.default_rng(90 + k + n1)
    q = (rng.integers(-20, 21, size=(B, n1, 3)) / 4).astype(np.float32)
    r = (rng.integers(-20, 21, size=(B, n2, 3)) / 4).astype(np.float32)
    d, i = knn_points(T(q), T(r), k, sorted=True)
    e, j = oracle.knn(q, r, k)
    np.testing.assert_array_equal(N(i), j)
    np.testing.assert_array_equal(N(d), e)


@pytest.mark.parametrize("k", [1, 2, 3, 4])
def test_knn_small_full_round_of_blocks_bit_exact(oracle, k):
    """Two queries per thread, about one full round of 256-query blocks per SM (1016 blocks), with ties."""
    from torkit3d_b200.ops import knn_points

    rng = np.random.default_rng(40 + k)
    q = (rng.integers(-30, 31, size=(2, 130000, 3)) / 8).astype(np.float32)   # lattice: many ties
    r = (rng.integers(-30, 31, size=(2, 3000, 3)) / 8).astype(np.float32)
    d, i = knn_points(T(q), T(r), k, sorted=True)
    e, j = oracle.knn(q, r, k)
    np.testing.assert_array_equal(N(i), j)
    np.testing.assert_array_equal(N(d), e)


# float64 with few queries: several warps per query group, per-segment lists merged at the end
@pytest.mark.parametrize("B,n1,n2,k", [(8, 2048, 2048, 16), (2, 100, 300, 16), (1, 33, 1000, 64), (3, 500, 257, 3),
                                       (2, 700, 5000, 1), (1, 40, 9000, 33)])
@pytest.mark.parametrize("ties", [False, True])
def test_knn_fp64_split_path_bit_exact(oracle, B, n1, n2, k, ties):
    from torkit3d_b200.ops import knn_points

    rng = np.random.default_rng(n2 + k)
    if ties:
        q, r = grid_cloud(rng, B, n1, np.float64), grid_cloud(rng, B, n2, np.float64)
    else:
        q, r = rng.standard_normal((B, n1, 3)), rng.standard_normal((B, n2, 3))
    d, i = knn_points(T(q), T(r), k, sorted=True)
    e, j = oracle.knn(q, r, k)
    np.testing.assert_array_equal(N(i), j)
    np.testing.assert_array_equal(N(d), e)


def test_knn_golden_fp64_and_options(golden):
    from torkit3d_b200.ops import knn_points

    g = golden("knn")
    for tag in "abc":
        k = int(g[tag + "_k"])
        q, r = T(g[tag + "_query"]), T(g[tag + "_key"])
        d, i = knn_points(q, r, k, sorted=True, sqrt_distance=True)
        np.testing.assert_array_equal(N(i), g[tag + "_idx"])
        np.testing.assert_allclose(N(d), g[tag + "_dist"], rtol=1e-4, atol=5e-5)
        for version in (0, 1):
            d2, i2 = knn_points(q.transpose(1, 2), r.transpose(1, 2), k, transpose=True, version=version)
            assert torch.equal(i2, i)
    with pytest.raises(RuntimeError):
        knn_points(q, r[:, :5], 31)
    with pytest.raises(RuntimeError, match="Invalid version"):
        knn_points(q, r, 3, version=2)


def test_knn_far_from_origin(oracle):
    from torkit3d_b200.ops import knn_points

    rng = np.random.default_rng(2)
    for k in (3, 16):
        q = (rng.standard_normal((2, 200, 3)) + 500.0).astype(np.float32)
        r = (rng.standard_normal((2, 800, 3)) + 500.0).astype(np.float32)
        d, i = knn_points(T(q), T(r), k)
        e, j = oracle.knn(q, r, k)
        np.testing.assert_array_equal(N(i), j)
        np.testing.assert_array_equal(N(d), e)


# ----------------------------------------------------------------------------- knn on features
FEATURE_KNN_SHAPES = [(2, 16, 300, 300, 20, True), (1, 67, 129, 257, 33, True), (3, 5, 64, 200, 7, False),
                      (1, 130, 40, 150, 70, True), (2, 64, 1024, 1024, 20, True), (1, 3, 100, 500, 128, False),
                      (4, 8, 33, 128, 1, True), (2, 40, 257, 129, 64, False)]


@pytest.mark.parametrize("B,C,n1,n2,k,cf", FEATURE_KNN_SHAPES)
@pytest.mark.parametrize("ties", [False, True])
def test_feature_knn_bit_exact(oracle, B, C, n1, n2, k, cf, ties):
    from torkit3d_b200 import _C

    rng = np.random.default_rng(C * 100 + n2 + k)
    shape_q, shape_r = ((B, C, n1), (B, C, n2)) if cf else ((B, n1, C), (B, n2, C))
    if ties:   # small integer lattice: many exactly equal distances, ties must go to the lower index
        q = rng.integers(-2, 3, size=shape_q).astype(np.float32)
        r = rng.integers(-2, 3, size=shape_r).astype(np.float32)
    else:
        q = rng.standard_normal(shape_q).astype(np.float32)
        r = rng.standard_normal(shape_r).astype(np.float32)
    d, i = [N(t) for t in _C.feature_knn_cuda(T(q), T(r), k, channel_first=cf)]
    e, j = oracle.feature_knn(q, r, k, channel_first=cf)
    np.testing.assert_array_equal(i, j)
    np.testing.assert_array_equal(d, e)


def test_feature_knn_golden_wrapper_and_errors(golden):
    from torkit3d_b200 import _C
    from torkit3d_b200.ops import knn

    g = golden("feature_knn")
    for tag in "abcd":
        k, cf = int(g[tag + "_k"]), bool(g[tag + "_cf"])
        q, r = T(g[tag + "_query"], torch.float32), T(g[tag + "_key"], torch.float32)
        d, i = knn(q, r, k, sorted=True, transpose=cf)
        assert (N(i) == g[tag + "_idx"]).mean() > 0.995
        np.testing.assert_allclose(N(d), g[tag + "_dist"], rtol=1e-5, atol=1e-6)
    # differentiable distances when an input requires grad; same neighbours
    q = T(g["a_query"], torch.float32).requires_grad_(True)
    r = T(g["a_key"], torch.float32)
    d, i = knn(q, r, 20, transpose=True)
    d0, i0 = knn(q.detach(), r, 20, transpose=True)
    assert torch.equal(i, i0)
    np.testing.assert_allclose(N(d), N(d0), rtol=1e-5, atol=1e-6)
    d.sum().backward()
    assert q.grad is not None and torch.isfinite(q.grad).all()
    with pytest.raises(RuntimeError):
        _C.feature_knn_cuda(r, r, 301)          # k > N2
    with pytest.raises(RuntimeError):
        _C.feature_knn_cuda(r, r.double(), 3)    # dtype mismatch
    with pytest.raises(RuntimeError):
        _C.feature_knn_cuda(r, r, 129)          # k beyond the kernel's list capacity
    # beyond that capacity the wrapper runs the reference formulation on the same device
    d, i = knn(r, r, 130, sorted=True, transpose=True)
    assert d.shape == (2, 300, 130) and i.is_cuda


# ----------------------------------------------------------------------------------------------- fps
FPS_CASES = [(1, 31, 2), (2, 1024, 128), (3, 1025, 129), (16, 1024, 512), (4, 4096, 300), (2, 8192, 1024),
             (2, 100, 100), (1, 1, 1), (3, 33, 33), (2, 8193, 200), (1, 20000, 64),
             # few clouds of 4097 to 16384 points: clusters of eight small blocks without barriers in the step;
             # many such clouds: one block per cloud again
             (2, 4097, 50), (3, 5000, 300), (1, 16384, 128), (40, 6000, 64), (3, 12345, 2000), (90, 4500, 32),
             # a cluster of 8 / 16 blocks per cloud (16385 to 262144 points; beyond 131072 the coordinates stay in
             # shared memory), then the streaming kernel
             (2, 16385, 96), (3, 30000, 128), (2, 40961, 70), (1, 65536, 200), (1, 65537, 40), (1, 131072, 33),
             (1, 131073, 20), (2, 200000, 30), (1, 262144, 16), (1, 262145, 8)]


@pytest.mark.parametrize("B,n,s", FPS_CASES)
def test_fps_bit_exact(oracle, B, n, s):
    from torkit3d_b200.ops import sample_farthest_points

    rng = np.random.default_rng(n + s)
    p = rng.random((B, n, 3)).astype(np.float32)
    got = N(sample_farthest_points(T(p), s))
    np.testing.assert_array_equal(got, oracle.fps(p, s))
    got_t = N(sample_farthest_points(T(p).transpose(1, 2), s, transpose=True))
    np.testing.assert_array_equal(got_t, got)


def test_fps_cluster_ties_and_gather(oracle):
    """Clouds served by a cluster of blocks: exact ties across the blocks' slices (a coarse lattice:
    the lowest index must win wherever it lives), all points coinciding, and the fused centroid
    gather in both layouts."""
    from torkit3d_b200 import _fused
    from torkit3d_b200.ops import sample_farthest_points

    rng = np.random.default_rng(77)
    p = (rng.integers(-6, 7, size=(2, 33000, 3)) * 0.5).astype(np.float32)
    np.testing.assert_array_equal(N(sample_farthest_points(T(p), 300)), oracle.fps(p, 300))
    same = np.full((1, 17000, 3), 0.25, dtype=np.float32)
    np.testing.assert_array_equal(N(sample_farthest_points(T(same), 5)), oracle.fps(same, 5))
    for n in (20000, 7000, 9001):  # 1024-thread blocks with a cluster barrier; eight blocks of 64 / 128 threads
        q = rng.random((2, n, 3)).astype(np.float32)
        want = oracle.fps(q, 64)
        for cf in (False, True):
            pts = T(q).transpose(1, 2).contiguous() if cf else T(q)
            idx, cent = _fused.fps_gather(pts, 64, channel_first=cf)
            np.testing.assert_array_equal(N(idx), want)
            ref = np.take_along_axis(q, want[..., None], axis=1)
            np.testing.assert_array_equal(N(cent.transpose(1, 2) if cf else cent), ref)
    # the same ties and coinciding points on the barrier-free kernel's sizes
    p = (rng.integers(-4, 5, size=(3, 8000, 3)) * 0.5).astype(np.float32)
    np.testing.assert_array_equal(N(sample_farthest_points(T(p), 400)), oracle.fps(p, 400))
    same = np.full((2, 10000, 3), -1.5, dtype=np.float32)
    np.testing.assert_array_equal(N(sample_farthest_points(T(same), 7)), oracle.fps(same, 7))
    dup = rng.random((1, 3000, 3)).astype(np.float32)
    dup = np.concatenate([dup, dup, dup[:, :500]], axis=1)  # every point twice or three times
    np.testing.assert_array_equal(N(sample_farthest_points(T(dup), 3200)), oracle.fps(dup, 3200))


@pytest.mark.parametrize("B,n,s", [(2, 3000, 60), (1, 4097, 40), (2, 8192, 50), (3, 9000, 30), (1, 20000, 40),
                                   (1, 40000, 20), (1, 70000, 16), (1, 131072, 10), (1, 131073, 6), (90, 2500, 16)])
def test_fps_float64_clusters_bit_exact(oracle, B, n, s):
    """float64 clouds on thread-block clusters (few clouds of 2049 to 8192 points, every cloud of 8193 to
    131072 points), the streaming kernel beyond, one block per cloud for large batches; both layouts."""
    from torkit3d_b200.ops import sample_farthest_points

    rng = np.random.default_rng(n + s)
    p = rng.random((B, n, 3))
    want = oracle.fps(p, s)
    np.testing.assert_array_equal(N(sample_farthest_points(T(p), s)), want)
    np.testing.assert_array_equal(N(sample_farthest_points(T(p).transpose(1, 2), s, transpose=True)), want)


def test_fps_float64_cluster_ties_and_gather(oracle):
    from torkit3d_b200 import _fused
    from torkit3d_b200.ops import sample_farthest_points

    rng = np.random.default_rng(78)
    p = rng.integers(-5, 6, size=(2, 6000, 3)) * 0.5  # a coarse lattice: exact ties across the blocks' slices
    np.testing.assert_array_equal(N(sample_farthest_points(T(p), 300)), oracle.fps(p, 300))
    same = np.full((1, 9000, 3), 0.25)
    np.testing.assert_array_equal(N(sample_farthest_points(T(same), 5)), oracle.fps(same, 5))
    q = rng.random((2, 12000, 3))
    want = oracle.fps(q, 48)
    for cf in (False, True):
        pts = T(q).transpose(1, 2).contiguous() if cf else T(q)
        idx, cent = _fused.fps_gather(pts, 48, channel_first=cf)
        np.testing.assert_array_equal(N(idx), want)
        ref = np.take_along_axis(q, want[..., None], axis=1)
        np.testing.assert_array_equal(N(cent.transpose(1, 2) if cf else cent), ref)


def test_fps_golden_fp64_and_duplicates(oracle, golden):
    from torkit3d_b200.ops import sample_farthest_points

    g = golden("fps")
    for tag in "abcd":
        got = N(sample_farthest_points(T(g[tag + "_points"]), int(g[tag + "_s"])))
        np.testing.assert_array_equal(got, g[tag + "_idx"])
    rng = np.random.default_rng(0)
    p = rng.random((2, 600, 3)).astype(np.float32)
    p = np.concatenate([p, p, p[:, :100]], axis=1)  # exact duplicates -> tied maxima
    for dtype in (np.float32, np.float64):
        np.testing.assert_array_equal(N(sample_farthest_points(T(p.astype(dtype)), 1300)), oracle.fps(p.astype(dtype), 1300))
    ones = torch.ones(2, 50, 3, device=DEV)
    assert (sample_farthest_points(ones, 20) == 0).all()
    with pytest.raises(RuntimeError):
        sample_farthest_points(ones, 51)
    with pytest.raises(RuntimeError):
        sample_farthest_points(ones, 0)


# ---------------------------------------------------------------------------------------- ball query
@pytest.mark.parametrize("B,n1,n2,r,k", [(2, 64, 128, 0.1, 32), (3, 65, 129, 10.0, 32), (4, 513, 2000, 0.3, 16),
                                        (2, 1000, 5000, 0.2, 64), (1, 1, 1, 1.0, 4), (2, 100, 700, 0.05, 1),
                                        (30, 300, 600, 0.4, 8), (40, 8000, 300, 0.4, 8)])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_ball_query_bit_exact(oracle, B, n1, n2, r, k, dtype):
    from torkit3d_b200.ops import ball_query

    rng = np.random.default_rng(n1 + k)
    key = rng.standard_normal((B, n2, 3)).astype(dtype)
    query = rng.standard_normal((B, n1, 3)).astype(dtype)
    h = min(n1 // 2, n2)
    query[:, :h] = key[:, :h]  # up to half of the queries coincide with keys
    got = N(ball_query(T(query), T(key), r, k, transpose=False))
    np.testing.assert_array_equal(got, oracle.ball_query(query, key, r, k))
    got_t = N(ball_query(T(query).transpose(1, 2), T(key).transpose(1, 2), r, k))  # default: channel-first
    np.testing.assert_array_equal(got_t, got)


def test_ball_query_golden_and_boundary(oracle, golden):
    from torkit3d_b200.ops import ball_query

    g = golden("ball_query")
    for tag in "abcd":
        got = N(ball_query(T(g[tag + "_query"]), T(g[tag + "_key"]), float(g[tag + "_r"]), int(g[tag + "_k"]),
                           transpose=False))
        np.testing.assert_array_equal(got, g[tag + "_idx"])
    # points exactly on the sphere are outside (strict "<"); grid data gives many such cases
    rng = np.random.default_rng(1)
    q, r = grid_cloud(rng, 2, 200), grid_cloud(rng, 2, 900)
    for radius in (0.25, 0.5, 0.75):
        got = N(ball_query(T(q), T(r), radius, 12, transpose=False))
        np.testing.assert_array_equal(got, oracle.ball_query(q, r, radius, 12))


# ------------------------------------------------------------------------------- group / interpolate
@pytest.mark.parametrize("B,C,n1,n2,k", [(2, 3, 512, 128, 32), (5, 64, 513, 129, 33), (1, 1, 1, 1, 1), (3, 7, 100, 50, 5),
                                        (4, 32, 2048, 512, 16), (2, 5, 260, 37, 31), (1, 4, 12288, 64, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_group_points(oracle, B, C, n1, n2, k, dtype):
    from torkit3d_b200.ops import group_points

    torch.manual_seed(0)
    f = torch.randn(B, C, n1, dtype=dtype, device=DEV, requires_grad=True)
    idx = torch.randint(0, n1, (B, n2, k), device=DEV)
    idx[:, :, k // 2:] = idx[:, :, :1]  # padded rows, as ball query produces them
    out = group_points(f, idx)
    np.testing.assert_array_equal(N(out), oracle.group_fwd(N(f), N(idx)))
    go = torch.randn_like(out)
    out.backward(go)
    ref = oracle.group_bwd(N(go).astype(np.float64), N(idx), n1)
    np.testing.assert_allclose(N(f.grad), ref, rtol=1e-5, atol=2e-5 if dtype == torch.float32 else 1e-12)


def test_group_golden_and_bad_index(golden):
    from torkit3d_b200 import _C, _lib
    from torkit3d_b200.ops import group_points

    g = golden("group_points")
    for tag in "ab":
        f = T(g[tag + "_feature"]).requires_grad_(True)
        out = group_points(f, T(g[tag + "_index"]))
        np.testing.assert_array_equal(N(out), g[tag + "_out"])
        out.backward(torch.ones_like(out))
        np.testing.assert_allclose(N(f.grad), g[tag + "_grad"], rtol=1e-6, atol=1e-6)
    # an index of -1 (ball query row without a hit) reads as zero and raises the status bit
    f = torch.randn(1, 2, 10, device=DEV)
    idx = torch.tensor([[[0, -1, 9, 10]]], device=DEV)
    out = _C.group_points_forward_cuda(f, idx)
    assert torch.equal(out[0, :, 0, 1], torch.zeros(2, device=DEV)) and torch.equal(out[0, :, 0, 3], torch.zeros(2, device=DEV))
    assert torch.equal(out[0, :, 0, 0], f[0, :, 0]) and torch.equal(out[0, :, 0, 2], f[0, :, 9])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    lib = _lib.load()
    o2 = torch.empty_like(out)
    assert lib.tk3d_group_fwd(f.data_ptr(), idx.data_ptr(), 1, 2, 10, 1, 4, o2.data_ptr(), status.data_ptr(), None, 0, 0,
                              torch.cuda.current_stream().cuda_stream) == 0
    assert int(status.item()) == 1 and torch.equal(o2, out)


@pytest.mark.parametrize("B,C,n1,n2", [(2, 64, 128, 512), (3, 65, 129, 513), (1, 1, 3, 1), (4, 128, 1000, 3000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_interpolate(oracle, B, C, n1, n2, dtype):
    from torkit3d_b200.ops import interpolate_feature

    torch.manual_seed(1)
    f = torch.randn(B, C, n1, dtype=dtype, device=DEV, requires_grad=True)
    idx = torch.randint(0, n1, (B, n2, 3), device=DEV)
    w = torch.rand(B, n2, 3, dtype=dtype, device=DEV)
    w = w / w.sum(2, keepdim=True)
    out = interpolate_feature(f, idx, w)
    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-12, atol=1e-14)
    np.testing.assert_allclose(N(out), oracle.interp_fwd(N(f).astype(np.float64), N(idx), N(w).astype(np.float64)), **tol)
    go = torch.randn_like(out)
    out.backward(go)
    ref = oracle.interp_bwd(N(go).astype(np.float64), N(idx), N(w).astype(np.float64), n1)
    np.testing.assert_allclose(N(f.grad), ref, rtol=1e-5, atol=2e-5 if dtype == torch.float32 else 1e-12)


def test_interpolate_golden_weights_and_errors(oracle, golden):
    from torkit3d_b200.ops import interpolate_feature, knn_points, three_nn_weight

    g = golden("interpolate")
    for tag in "ab":
        f = T(g[tag + "_feature"]).requires_grad_(True)
        out = interpolate_feature(f, T(g[tag + "_index"]), T(g[tag + "_weight"]))
        np.testing.assert_allclose(N(out), g[tag + "_out"], rtol=1e-12, atol=1e-14)
        out.backward(torch.ones_like(out))
        np.testing.assert_allclose(N(f.grad), g[tag + "_grad"], rtol=1e-10, atol=1e-12)
    with pytest.raises(RuntimeError, match="k=3"):
        interpolate_feature(torch.randn(1, 2, 8, device=DEV), torch.zeros(1, 4, 2, dtype=torch.long, device=DEV),
                            torch.ones(1, 4, 2, device=DEV))
    # three-NN chain: knn (k=3) -> weights -> interpolate, against the oracle chain
    rng = np.random.default_rng(5)
    q = rng.random((2, 700, 3)).astype(np.float32)
    r = rng.random((2, 300, 3)).astype(np.float32)
    r[0, 0] = q[0, 0]  # a zero distance exercises the clamp
    feat = rng.standard_normal((2, 16, 300)).astype(np.float32)
    d, i = knn_points(T(q), T(r), 3)
    w = three_nn_weight(d)
    ed, ei = oracle.knn(q, r, 3)
    ew = oracle.three_nn_weight(ed)
    np.testing.assert_array_equal(N(i), ei)
    np.testing.assert_allclose(N(w), ew, rtol=1e-6)
    out = interpolate_feature(T(feat), i, w)
    np.testing.assert_allclose(N(out), oracle.interp_fwd(feat, ei, ew), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("B,C,n1,n2,k", [(3, 64, 700, 300, 16), (2, 33, 129, 100, 9), (2, 128, 512, 2048, 4), (1, 512, 64, 70, 5),
                                        (2, 64, 40, 25, 4), (2, 96, 100, 333, 12), (1, 512, 100, 201, 4)])
def test_group_and_interp_row_gather_path_equals_direct_path(oracle, B, C, n1, n2, k):
    """With a scratch buffer the forward gathers run on transposed features; same results."""
    from torkit3d_b200 import _lib

    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(3)
    f = torch.randn(B, C, n1, device=DEV)
    idx = torch.randint(0, n1, (B, n2, k), device=DEV)
    idx[0, 0, 0] = -1  # bad index: reads as zero on both paths
    need = lib.tk3d_group_fwd_scratch_bytes(B, C, n1, n2, k, 0)
    # shapes served by the channel-row kernel (rows staged in shared memory) need no scratch at all
    assert need in (0, B * C * n1 * 4)
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o_rows = torch.full((B, C, n2, k), float("nan"), device=DEV)
    o_direct = torch.full((B, C, n2, k), float("nan"), device=DEV)
    assert lib.tk3d_group_fwd(f.data_ptr(), idx.data_ptr(), B, C, n1, n2, k, o_rows.data_ptr(), status.data_ptr(),
                              scratch.data_ptr(), need, 0, st) == 0
    assert lib.tk3d_group_fwd(f.data_ptr(), idx.data_ptr(), B, C, n1, n2, k, o_direct.data_ptr(), None, None, 0, 0, st) == 0
    assert torch.equal(o_rows, o_direct) and int(status.item()) == 1
    ref_idx = idx.clone()
    ref_idx[0, 0, 0] = 0
    ref = oracle.group_fwd(N(f), N(ref_idx))
    ref[0, :, 0, 0] = 0
    np.testing.assert_array_equal(N(o_rows), ref)
    # interpolation: k=3 neighbours
    idx3 = torch.randint(0, n1, (B, n2, 3), device=DEV)
    w = torch.rand(B, n2, 3, device=DEV)
    need3 = lib.tk3d_interp_fwd_scratch_bytes(B, C, n1, n2, 0)
    i_rows = torch.full((B, C, n2), float("nan"), device=DEV)
    i_direct = torch.full((B, C, n2), float("nan"), device=DEV)
    if need3:
        scratch3 = torch.empty(need3, dtype=torch.uint8, device=DEV)
        assert lib.tk3d_interp_fwd(f.data_ptr(), idx3.data_ptr(), w.data_ptr(), B, C, n1, n2, 3, i_rows.data_ptr(), None,
                                   scratch3.data_ptr(), need3, 0, st) == 0
        assert lib.tk3d_interp_fwd(f.data_ptr(), idx3.data_ptr(), w.data_ptr(), B, C, n1, n2, 3, i_direct.data_ptr(), None,
                                   None, 0, 0, st) == 0
        torch.testing.assert_close(i_rows, i_direct, rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(N(i_rows), oracle.interp_fwd(N(f), N(idx3), N(w)), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("B,C,n1,n2,k", [(2, 64, 300, 700, 32), (2, 33, 129, 100, 9), (1, 512, 64, 40, 16),
                                         (3, 16, 1000, 222, 4), (2, 128, 4100, 9000, 3)])
@pytest.mark.parametrize("index_dtype", [torch.int64, torch.int32])
def test_features_kept_as_rows(oracle, B, C, n1, n2, k, index_dtype):
    """``feature_rows`` once, then gathers that skip their own transposition: same results as the
    operators on the [B,C,N1] tensor, for sizes that take the 16-byte kernels and sizes that do not,
    with both index types, and the same gradient for the features."""
    from torkit3d_b200 import _C
    from torkit3d_b200.ops import feature_rows, group_points, interpolate_feature

    g = torch.Generator().manual_seed(C + n2)
    f = torch.randn(B, C, n1, generator=g).to(DEV)
    rows = feature_rows(f)
    assert rows.shape == (B, n1, C) and torch.equal(rows, f.transpose(1, 2).contiguous())
    idx = torch.randint(0, n1, (B, n2, k), generator=g).to(DEV)
    out = _C.group_points_forward_rows_cuda(rows, idx.to(index_dtype))
    np.testing.assert_array_equal(N(out), oracle.group_fwd(N(f), N(idx)))
    idx3 = torch.randint(0, n1, (B, n2, 3), generator=g).to(DEV)
    w = torch.rand(B, n2, 3, generator=g).to(DEV)
    o3 = _C.interpolate_forward_rows_cuda(rows, idx3.to(index_dtype), w)
    np.testing.assert_allclose(N(o3), oracle.interp_fwd(N(f), N(idx3), N(w)), rtol=1e-5, atol=1e-6)
    # through the operators, with gradients
    fa = f.clone().requires_grad_(True)
    fb = f.clone().requires_grad_(True)
    ya = interpolate_feature(fa, idx3, w, rows=rows) .sum() + group_points(fa, idx, rows=rows).square().sum()
    yb = interpolate_feature(fb, idx3, w).sum() + group_points(fb, idx).square().sum()
    ya.backward()
    yb.backward()
    torch.testing.assert_close(ya, yb, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(fa.grad, fb.grad, rtol=1e-5, atol=1e-5)


def test_features_kept_as_rows_errors():
    from torkit3d_b200 import _C

    f = torch.randn(2, 8, 50, device=DEV)
    rows = _C.feature_rows(f)
    with pytest.raises(RuntimeError):
        _C.feature_rows(f.double())
    with pytest.raises(RuntimeError):
        _C.feature_rows(f.cpu())
    with pytest.raises(RuntimeError):
        _C.group_points_forward_rows_cuda(rows, torch.zeros(3, 4, 5, dtype=torch.int64, device=DEV))
    with pytest.raises(RuntimeError):
        _C.interpolate_forward_rows_cuda(rows, torch.zeros(2, 4, 2, dtype=torch.int64, device=DEV),
                                         torch.zeros(2, 4, 2, device=DEV))
    # an out-of-range index gathers zeros (and is reported through the C ABI's status word)
    idx = torch.full((2, 4, 5), 50, dtype=torch.int64, device=DEV)
    assert float(_C.group_points_forward_rows_cuda(rows, idx).abs().max()) == 0.0


@pytest.mark.parametrize("B,C,n1,n2,k", [(3, 64, 700, 300, 16), (2, 128, 512, 2048, 4), (2, 64, 40, 25, 4), (2, 96, 100, 333, 12)])
def test_group_and_interp_backward_row_path_equals_direct_path(oracle, B, C, n1, n2, k):
    """With scratch the backward accumulates into a transposed buffer with vector atomics; same sums."""
    from torkit3d_b200 import _lib

    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(4)
    idx = torch.randint(0, n1, (B, n2, k), device=DEV)
    idx[:, :, k // 2:] = idx[:, :, :1]
    idx[0, 0, 0] = n1 + 5  # out of range: skipped on both paths
    go = torch.randn(B, C, n2, k, device=DEV)
    need = lib.tk3d_group_bwd_scratch_bytes(B, C, n1, n2, k, 0)
    assert need == B * C * n1 * 4
    scratch = torch.full((need,), 77, dtype=torch.uint8, device=DEV)  # contents must be ignored
    g_rows = torch.full((B, C, n1), float("nan"), device=DEV)
    g_direct = torch.full((B, C, n1), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert lib.tk3d_group_bwd(go.data_ptr(), idx.data_ptr(), B, C, n1, n2, k, g_rows.data_ptr(), status.data_ptr(),
                              scratch.data_ptr(), need, 0, st) == 0
    assert lib.tk3d_group_bwd(go.data_ptr(), idx.data_ptr(), B, C, n1, n2, k, g_direct.data_ptr(), None, None, 0, 0, st) == 0
    assert int(status.item()) == 1
    torch.testing.assert_close(g_rows, g_direct, rtol=1e-5, atol=2e-5)
    ref_idx = idx.clone()
    ref_idx[0, 0, 0] = 0
    gz = go.clone()
    gz[0, :, 0, 0] = 0
    np.testing.assert_allclose(N(g_rows), oracle.group_bwd(N(gz).astype(np.float64), N(ref_idx), n1), rtol=1e-5, atol=2e-5)
    # interpolation backward (needs n2 % 4 == 0 for the row path)
    idx3 = torch.randint(0, n1, (B, n2, 3), device=DEV)
    w = torch.rand(B, n2, 3, device=DEV)
    go3 = torch.randn(B, C, n2, device=DEV)
    need3 = lib.tk3d_interp_bwd_scratch_bytes(B, C, n1, n2, 0)
    i_direct = torch.empty(B, C, n1, device=DEV)
    assert lib.tk3d_interp_bwd(go3.data_ptr(), idx3.data_ptr(), w.data_ptr(), B, C, n1, n2, 3, i_direct.data_ptr(), None,
                               None, 0, 0, st) == 0
    if need3:
        scratch3 = torch.empty(need3, dtype=torch.uint8, device=DEV)
        i_rows = torch.empty(B, C, n1, device=DEV)
        assert lib.tk3d_interp_bwd(go3.data_ptr(), idx3.data_ptr(), w.data_ptr(), B, C, n1, n2, 3, i_rows.data_ptr(), None,
                                   scratch3.data_ptr(), need3, 0, st) == 0
        torch.testing.assert_close(i_rows, i_direct, rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(N(i_direct), oracle.interp_bwd(N(go3).astype(np.float64), N(idx3), N(w).astype(np.float64), n1),
                               rtol=1e-5, atol=2e-5)


def test_non_default_stream_and_determinism():
    """Index results are identical run to run and on a side stream."""
    from torkit3d_b200.ops import knn_points, nn_distance, sample_farthest_points

    torch.manual_seed(0)
    a = torch.randn(4, 2000, 3, device=DEV)
    b = torch.randn(4, 1500, 3, device=DEV)
    base = nn_distance(a, b)
    kb = knn_points(a, b, 16)
    fb = sample_farthest_points(a, 256)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        again = nn_distance(a, b)
        ka = knn_points(a, b, 16)
        fa = sample_farthest_points(a, 256)
    s.synchronize()
    for x, y in zip(base, again):
        assert torch.equal(x, y)
    assert torch.equal(kb[0], ka[0]) and torch.equal(kb[1], ka[1]) and torch.equal(fa, fb)
