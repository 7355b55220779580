"""Parity against the REFERENCE's own CUDA extension, compiled unmodified with -fmad=false
(oracle/build_ref.py -> oracle/_ref/nofma/_C.so).  Skipped when that build is not present.

KNN rows of the reference come in an unspecified slot order and are canonicalised by sorting on
(distance, index) before the bit-exact comparison."""
import importlib.util
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "nofma", "_C.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO):
        pytest.skip("reference CUDA extension not built (python oracle/build_ref.py --ref <checkout>)")
    spec = importlib.util.spec_from_file_location("_C", REF_SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def canon(dist, idx):
    d, i = dist.cpu().numpy(), idx.cpu().numpy()
    order = np.lexsort((i, d), axis=-1)
    return np.take_along_axis(d, order, -1), np.take_along_axis(i, order, -1)


def test_chamfer(ref):
    from torkit3d_b200 import _C, workloads

    for x1, x2 in (workloads.c1_chamfer_small(), workloads.c4_chamfer_large(num_clouds=4),
                   (torch.randn(3, 1000, 3), torch.randn(3, 777, 3))):
        a, b = x1.to(DEV), x2.to(DEV)
        mine = _C.chamfer_distance_forward_cuda(a, b)
        theirs = ref.chamfer_distance_forward_cuda(a, b)
        for m, t in zip(mine, theirs):
            assert torch.equal(m, t)
        g1, g2 = torch.randn_like(mine[0]), torch.randn_like(mine[2])
        gm = _C.chamfer_distance_backward_cuda(g1, g2, a, b, mine[1], mine[3])
        gt = ref.chamfer_distance_backward_cuda(g1, g2, a, b, theirs[1], theirs[3])
        for m, t in zip(gm, gt):
            torch.testing.assert_close(m, t, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("k,version", [(3, 1), (16, 1), (32, 1), (64, 1), (31, 0), (5, 0), (130, 0)])
def test_knn(ref, k, version):
    from torkit3d_b200 import _C, workloads

    q, r = workloads.c2_knn(B=4, N1=1500, N2=2500)
    q, r = q.to(DEV), r.to(DEV)
    md, mi = _C.knn_distance_cuda(q, r, k, version)
    td, ti = ref.knn_distance_cuda(q, r, k, version)
    cd, ci = canon(td, ti)
    np.testing.assert_array_equal(mi.cpu().numpy(), ci)
    np.testing.assert_array_equal(md.cpu().numpy(), cd)


def test_fps_ball_group(ref):
    from torkit3d_b200 import _C, workloads

    p, feat = workloads.c3_set_abstraction(B=8)
    p, feat = p.to(DEV), feat.to(DEV)
    mi = _C.sample_farthest_points_cuda(p, 1024)
    ti = ref.sample_farthest_points_cuda(p, 1024)
    assert torch.equal(mi, ti)
    cent = torch.gather(p, 1, mi.unsqueeze(2).expand(-1, -1, 3)).contiguous()
    mb = _C.ball_query_cuda(cent, p, 0.1, 32)
    tb = ref.ball_query_cuda(cent, p, 0.1, 32)
    assert torch.equal(mb, tb)
    mg = _C.group_points_forward_cuda(feat, mb)
    tg = ref.group_points_forward_cuda(feat, tb)
    assert torch.equal(mg, tg)
    go = torch.randn_like(mg)
    torch.testing.assert_close(_C.group_points_backward_cuda(go, mb, 8192), ref.group_points_backward_cuda(go, tb, 8192),
                               rtol=1e-5, atol=2e-5)


def test_fps_double_and_odd_sizes(ref):
    from torkit3d_b200 import _C

    torch.manual_seed(0)
    for B, n, s, dt in ((3, 1025, 129, torch.float64), (2, 5000, 300, torch.float32), (2, 9000, 100, torch.float32)):
        p = torch.rand(B, n, 3, dtype=dt, device=DEV)
        assert torch.equal(_C.sample_farthest_points_cuda(p, s), ref.sample_farthest_points_cuda(p, s))


def test_interpolate(ref):
    from torkit3d_b200 import _C, workloads

    q, r, feat = workloads.c5_scene_interp(B=2, NQ=20000, NR=5000, C=32)
    q, r, feat = q.to(DEV), r.to(DEV), feat.to(DEV)
    md, mi = _C.knn_distance_cuda(q, r, 3, 1)
    td, ti = ref.knn_distance_cuda(q, r, 3, 1)
    cd, ci = canon(td, ti)
    np.testing.assert_array_equal(mi.cpu().numpy(), ci)
    np.testing.assert_array_equal(md.cpu().numpy(), cd)
    w = _C.three_nn_weight_cuda(md)
    inv = 1.0 / torch.clamp(md, min=1e-10)
    torch.testing.assert_close(w, inv / inv.sum(2, keepdim=True), rtol=1e-6, atol=0)
    mo = _C.interpolate_forward_cuda(feat, mi, w)
    to = ref.interpolate_forward_cuda(feat, mi, w)
    torch.testing.assert_close(mo, to, rtol=1e-5, atol=1e-6)
    go = torch.randn_like(mo)
    torch.testing.assert_close(_C.interpolate_backward_cuda(go, mi, w, 5000), ref.interpolate_backward_cuda(go, mi, w, 5000),
                               rtol=1e-5, atol=2e-5)


def test_full_size_chamfer_batch(ref):
    """All 64 cloud pairs of the 16384-point batch: distances and indices of both directions equal the
    reference extension's, element for element."""
    from torkit3d_b200 import _C, workloads

    x1, x2 = workloads.c4_chamfer_large()
    a, b = x1.to(DEV), x2.to(DEV)
    mine = _C.chamfer_distance_forward_cuda(a, b)
    theirs = ref.chamfer_distance_forward_cuda(a, b)
    for m, t in zip(mine, theirs):
        assert torch.equal(m, t)


def test_full_size_scene_three_nn(ref):
    """All 8 x 131072 queries of the scene-scale three-NN search against the reference extension (k=3,
    version 1), rows canonicalised by (distance, index) on the GPU."""
    from torkit3d_b200 import _C, workloads

    q, r, _ = workloads.c5_scene_interp(C=1)
    q, r = q.to(DEV), r.to(DEV)
    md, mi = _C.knn_distance_cuda(q, r, 3, 1)
    td, ti = ref.knn_distance_cuda(q, r, 3, 1)
    # canonical order on the device: sort by index, then stably by distance
    o = torch.argsort(ti, dim=2, stable=True)
    td, ti = torch.gather(td, 2, o), torch.gather(ti, 2, o)
    o = torch.argsort(td, dim=2, stable=True)
    td, ti = torch.gather(td, 2, o), torch.gather(ti, 2, o)
    assert torch.equal(mi, ti)
    assert torch.equal(md, td)


def test_knn_largest_shape_of_the_reference_tests(ref):
    """(32, 2048, 8192, k=64): the largest case of the reference's tests/ops/test_knn_distance.py, here in
    float32 against the reference extension (its own test runs it in float64 against cdist + topk)."""
    from torkit3d_b200 import _C

    g = torch.Generator().manual_seed(0)
    q = torch.randn(32, 2048, 3, generator=g).to(DEV)
    r = torch.randn(32, 8192, 3, generator=g).to(DEV)
    md, mi = _C.knn_distance_cuda(q, r, 64, 1)
    td, ti = ref.knn_distance_cuda(q, r, 64, 1)
    cd, ci = canon(td, ti)
    np.testing.assert_array_equal(mi.cpu().numpy(), ci)
    np.testing.assert_array_equal(md.cpu().numpy(), cd)


def test_random_shapes(ref):
    """Seeded random shapes, sizes and point distributions (uniform, normal, a coarse lattice with
    massive ties, a nearly flat slab) through every kernel choice of the KNN, ball-query and FPS
    dispatch -- among them radix selection for large k, the hit-mask ball query for few queries and
    the cluster FPS for large clouds -- against the reference's kernels."""
    import random

    from torkit3d_b200 import _C

    rnd = random.Random(1234)
    g = torch.Generator().manual_seed(5)

    def cloud(B, n, kind):
        if kind == 0:
            return torch.rand(B, n, 3, generator=g)
        if kind == 1:
            return torch.randn(B, n, 3, generator=g)
        if kind == 2:
            return torch.randint(-4, 5, (B, n, 3), generator=g) * 0.25
        return torch.rand(B, n, 3, generator=g) * torch.tensor([10.0, 10.0, 0.01])

    for _ in range(40):
        kind = rnd.randrange(4)
        B = rnd.choice([1, 2, 3, 5])
        n1 = rnd.choice([1, 17, 100, 333, 1000, 2500])
        n2 = rnd.choice([40, 257, 300, 1000, 3000, 9000])
        k = min(n2, rnd.choice([1, 3, 5, 16, 31, 41, 64, 65, 100, 130, 200, 256]))
        q, r = cloud(B, n1, kind).to(DEV), cloud(B, n2, kind).to(DEV)
        md, mi = _C.knn_distance_cuda(q, r, k, 0)
        cd, ci = canon(*ref.knn_distance_cuda(q, r, k, 0))
        np.testing.assert_array_equal(md.cpu().numpy(), cd, err_msg="knn %s" % ((kind, B, n1, n2, k),))
        if kind != 2:  # among exactly tied distances the reference's retained set is not the lowest indices
            np.testing.assert_array_equal(mi.cpu().numpy(), ci, err_msg="knn %s" % ((kind, B, n1, n2, k),))
        radius, K = rnd.choice([0.05, 0.2, 0.5, 1.5]), rnd.choice([1, 8, 32, 64, 128, 300])
        assert torch.equal(_C.ball_query_cuda(q, r, radius, K), ref.ball_query_cuda(q, r, radius, K)), \
            "ball query %s" % ((kind, B, n1, n2, radius, K),)
    for _ in range(8):
        kind = rnd.choice([0, 1, 3])  # exact ties are broken differently by the reference (lowest thread)
        B, n = rnd.choice([1, 2, 3]), rnd.choice([16385, 20000, 33333, 65536, 70000, 131072])
        s = rnd.choice([1, 7, 64, 200])
        p = cloud(B, n, kind).to(DEV)
        assert torch.equal(_C.sample_farthest_points_cuda(p, s), ref.sample_farthest_points_cuda(p, s)), \
            "fps %s" % ((kind, B, n, s),)
