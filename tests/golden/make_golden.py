"""Generate the golden fixtures in this directory from the REFERENCE's own Python code.

The reference (torkit3d) stores no golden vectors; what pins its operators are the brute-force
formulations inside its test files and ``torkit3d.ops.native.knn``.  This script imports exactly
those functions from a reference checkout (its CUDA extension is not needed: ``torkit3d._C`` is
replaced by an empty stub module so that the test files import), runs them on small seeded inputs
and stores inputs and outputs as ``.npz`` files.  The CPU oracle is then checked against these
files by tests/test_oracle_golden.py, and the CUDA library against both.

    python tests/golden/make_golden.py --ref /path/to/torkit3d-checkout

Functions used (paths inside the reference):
    tests/ops/test_chamfer_distance.py     nn_distance_torch, bpdist2
    torkit3d/ops/native.py                 knn
    tests/ops/test_sample_farthest_points.py  sample_farthest_points_np
    tests/ops/test_ball_query.py           ball_query_np
    tests/ops/test_group_points.py         group_points_builtin
    tests/ops/test_interpolate_feature.py  group_points_torch (+ the weighted sum of :19-21)

Callers of the operators (fixtures ``sa_group``, ``edge_feature``, ``fps_gather``, ``three_nn_interp``):
the reference's own modules and functions run unmodified --
    torkit3d/layers/pointnet2.py           SetAbstraction.forward (its MLP replaced by a module that
                                           records its input), FeatureInterpolator.forward
    torkit3d/ops/edge_conv.py              get_edge_feature_builtin, get_edge_feature_custom
    torkit3d/ops/sample_farthest_points.py + torkit3d/nn/functional.py  sample_farthest_points, batch_index_select
-- on top of a ``torkit3d._C`` whose entry points are filled with the brute-force formulations
listed above (``knn_distance_cuda``: ``native.knn`` evaluated in float64).  The stand-in for
``knn_distance_cuda`` accepts the channel-first tensors ``FeatureInterpolator`` passes (the real
extension rejects them, see the module's missing ``transpose=True``) and transposes them itself.
"""
import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_reference(ref):
    sys.path.insert(0, ref)
    import torkit3d  # noqa: F401  (pure-python package root)

    stub = types.ModuleType("torkit3d._C")
    sys.modules["torkit3d._C"] = stub
    torkit3d._C = stub

    def load(name):
        path = os.path.join(ref, "tests", "ops", name + ".py")
        spec = importlib.util.spec_from_file_location("ref_" + name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    mods = {n: load(n) for n in ("test_chamfer_distance", "test_sample_farthest_points", "test_ball_query",
                                 "test_group_points", "test_interpolate_feature")}
    from torkit3d.ops.native import knn as native_knn

    # torkit3d._C entry points expressed with the reference's own brute-force code
    def ball_query_cuda(query, key, radius, k):
        idx = mods["test_ball_query"].ball_query_np(query.numpy(), key.numpy(), radius, k, transpose=False)
        return torch.from_numpy(idx.astype(np.int64))

    def fps_cuda(points, s):
        return torch.from_numpy(mods["test_sample_farthest_points"].sample_farthest_points_np(points.numpy(), s)
                                .astype(np.int64))

    def knn_distance_cuda(query, key, k, version):
        if query.size(1) == 3 and query.size(2) != 3:  # channel-first, as FeatureInterpolator passes them
            query, key = query.transpose(1, 2), key.transpose(1, 2)
        d, i = native_knn(query.double(), key.double(), k, sorted=True)
        return (d * d).to(query.dtype), i

    def interpolate_forward_cuda(feature, index, weight):
        nb = mods["test_interpolate_feature"].group_points_torch(feature, index)
        return (nb * weight.unsqueeze(1)).sum(dim=-1)

    stub.ball_query_cuda = ball_query_cuda
    stub.sample_farthest_points_cuda = fps_cuda
    stub.knn_distance_cuda = knn_distance_cuda
    stub.interpolate_forward_cuda = interpolate_forward_cuda
    stub.group_points_forward_cuda = lambda f, i: mods["test_group_points"].group_points_builtin(f, i)
    return mods, native_knn


class _Capture(torch.nn.Module):
    """Stands in for SetAbstraction.mlp: records the tensor that enters the MLP."""

    def forward(self, x):
        self.seen = x
        return x


def callers():
    """Fixtures of the layer code that calls the operators (run after _load_reference)."""
    from torkit3d.layers.pointnet2 import BallQuery, FeatureInterpolator, SetAbstraction
    from torkit3d.nn.functional import batch_index_select
    from torkit3d.ops.edge_conv import get_edge_feature_builtin, get_edge_feature_custom
    from torkit3d.ops.sample_farthest_points import sample_farthest_points

    def sphere(b, n, seed):
        g = torch.Generator().manual_seed(seed)
        p = torch.randn(b, n, 3, generator=g)
        return (p / p.norm(dim=2, keepdim=True) + 0.01 * torch.randn(b, n, 3, generator=g)).contiguous()

    # ---- FPS + centroid gather (models/classification/pointnet2.py:73-74) ----
    out = {}
    for tag, (b, n, s) in {"a": (2, 500, 64), "b": (3, 257, 33)}.items():
        pts = sphere(b, n, 100).transpose(1, 2).contiguous()  # [B,3,N]
        idx = sample_farthest_points(pts, s, True)
        xyz = batch_index_select(pts, idx, dim=2)
        out.update({tag + "_points": pts.numpy(), tag + "_index": idx.numpy(), tag + "_xyz": xyz.numpy(),
                    tag + "_s": np.int64(s)})
    np.savez_compressed(os.path.join(HERE, "fps_gather.npz"), **out)

    # ---- SetAbstraction.forward up to its MLP ----
    out = {}
    cases = {"a": (2, 400, 64, 16, 0.3, 16, True), "b": (2, 300, 40, 6, 0.35, 10, True),
             "c": (1, 256, 32, 0, 0.4, 8, True), "d": (2, 256, 48, 8, 0.3, 12, False)}
    for tag, (b, n, m, c, radius, k, use_xyz) in cases.items():
        pts = sphere(b, n, 200)
        g = torch.Generator().manual_seed(201)
        cen = pts[:, torch.randperm(n, generator=g)[:m]].contiguous()
        feat = torch.randn(b, c, n, generator=g) if c else None
        sa = SetAbstraction(c, [4], BallQuery(radius, k), use_xyz)
        sa.mlp = _Capture()
        in_xyz, out_xyz = pts.transpose(1, 2).contiguous(), cen.transpose(1, 2).contiguous()
        sa(in_xyz, out_xyz, feat)
        out.update({tag + "_in_xyz": in_xyz.numpy(), tag + "_out_xyz": out_xyz.numpy(),
                    tag + "_nbr": sa.mlp.seen.numpy(), tag + "_radius": np.float64(radius), tag + "_k": np.int64(k),
                    tag + "_use_xyz": np.int64(use_xyz)})
        if c:
            out[tag + "_feature"] = feat.numpy()
    np.savez_compressed(os.path.join(HERE, "sa_group.npz"), **out)

    # ---- EdgeConv edge features ----
    out = {}
    for tag, (b, c, n1, n2, k) in {"a": (2, 8, 128, 128, 20), "b": (2, 6, 50, 70, 7)}.items():
        g = torch.Generator().manual_seed(300)
        q = torch.randn(b, c, n1, generator=g)
        kf = torch.randn(b, c, n2, generator=g)
        idx = torch.randint(0, n2, (b, n1, k), generator=g)
        e0 = get_edge_feature_builtin(q, kf, idx)
        e1 = get_edge_feature_custom(q, kf, idx)
        assert torch.equal(e0, e1)
        out.update({tag + "_query": q.numpy(), tag + "_key": kf.numpy(), tag + "_index": idx.numpy(),
                    tag + "_edge": e0.numpy(), tag + "_edge_noquery": get_edge_feature_builtin(q, kf, idx, False).numpy()})
    np.savez_compressed(os.path.join(HERE, "edge_feature.npz"), **out)

    # ---- FeatureInterpolator.forward ----
    out = {}
    for tag, (b, nq, nk, c) in {"a": (2, 300, 100, 16), "b": (1, 129, 65, 5)}.items():
        g = torch.Generator().manual_seed(400)
        q = torch.rand(b, 3, nq, generator=g)
        kx = torch.rand(b, 3, nk, generator=g)
        f = torch.randn(b, c, nk, generator=g)
        o = FeatureInterpolator()(q, kx, f)
        out.update({tag + "_query": q.numpy(), tag + "_key": kx.numpy(), tag + "_feature": f.numpy(),
                    tag + "_out": o.numpy()})
    np.savez_compressed(os.path.join(HERE, "three_nn_interp.npz"), **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True)
    a = ap.parse_args()
    mods, native_knn = _load_reference(os.path.abspath(a.ref))

    # ---- chamfer: forward values/indices and autograd gradients of mean(dist1)+mean(dist2) ----
    out = {}
    for tag, (B, N, M, dt) in {"f32": (2, 128, 100, torch.float32), "f64": (2, 64, 64, torch.float64)}.items():
        g = torch.Generator().manual_seed(0)
        x1 = (torch.rand(B, N, 3, generator=g, dtype=dt) * 2 - 1).requires_grad_(True)
        x2 = (torch.rand(B, M, 3, generator=g, dtype=dt) * 2 - 1).requires_grad_(True)
        ref = mods["test_chamfer_distance"]
        d1, i1, d2, i2 = ref.nn_distance_torch(x1, x2)
        (d1.mean() + d2.mean()).backward()
        out.update({tag + "_xyz1": x1.detach().numpy(), tag + "_xyz2": x2.detach().numpy(),
                    tag + "_dist1": d1.detach().numpy(), tag + "_idx1": i1.numpy(),
                    tag + "_dist2": d2.detach().numpy(), tag + "_idx2": i2.numpy(),
                    tag + "_grad1": x1.grad.numpy(), tag + "_grad2": x2.grad.numpy()})
    np.savez_compressed(os.path.join(HERE, "chamfer.npz"), **out)

    # ---- knn: float64 inputs, as the reference test does, Euclidean distances, sorted ----
    out = {}
    for tag, (b, n1, n2, k) in {"a": (1, 512, 1024, 3), "b": (3, 511, 1025, 31), "c": (2, 100, 300, 16)}.items():
        torch.manual_seed(0)
        q = torch.randn(b, n1, 3).double()
        r = torch.randn(b, n2, 3).double()
        dist, idx = native_knn(q, r, k, sorted=True)
        out.update({tag + "_query": q.numpy(), tag + "_key": r.numpy(), tag + "_dist": dist.numpy(),
                    tag + "_idx": idx.numpy(), tag + "_k": np.int64(k)})
    np.savez_compressed(os.path.join(HERE, "knn.npz"), **out)

    # ---- knn on C-dimensional features, [B, C, N] tensors as DGCNN holds them (transpose=True), and
    # [B, N, C]; float64 so that cdist's own rounding cannot reorder neighbours ----
    out = {}
    for tag, (b, c, n1, n2, k, cf) in {"a": (2, 16, 300, 300, 20, True), "b": (1, 67, 129, 257, 33, True),
                                       "c": (3, 5, 64, 200, 7, False), "d": (1, 130, 40, 150, 70, True)}.items():
        torch.manual_seed(11)
        q = torch.randn(b, c, n1).double() if cf else torch.randn(b, n1, c).double()
        r = torch.randn(b, c, n2).double() if cf else torch.randn(b, n2, c).double()
        dist, idx = native_knn(q, r, k, sorted=True, transpose=cf)
        out.update({tag + "_query": q.numpy(), tag + "_key": r.numpy(), tag + "_dist": dist.numpy(),
                    tag + "_idx": idx.numpy(), tag + "_k": np.int64(k), tag + "_cf": np.int64(cf)})
    np.savez_compressed(os.path.join(HERE, "feature_knn.npz"), **out)

    # ---- fps ----
    out = {}
    for tag, (b, n, s, dt) in {"a": (1, 31, 2, np.float64), "b": (3, 1025, 129, np.float64),
                               "c": (2, 1024, 128, np.float64), "d": (2, 777, 200, np.float32)}.items():
        np.random.seed(0)
        p = np.random.rand(b, n, 3).astype(dt)
        idx = mods["test_sample_farthest_points"].sample_farthest_points_np(p, s)
        out.update({tag + "_points": p, tag + "_idx": idx.astype(np.int64), tag + "_s": np.int64(s)})
    np.savez_compressed(os.path.join(HERE, "fps.npz"), **out)

    # ---- ball query (queries are a subset of the keys, as in the reference test) ----
    out = {}
    for tag, (b, n1, n2, r, k) in {"a": (2, 64, 128, 0.1, 32), "b": (3, 65, 129, 0.1, 32),
                                   "c": (3, 65, 129, 10.0, 32), "d": (2, 40, 300, 0.5, 8)}.items():
        np.random.seed(0)
        key = np.random.randn(b, n2, 3)
        query = np.array([p[np.random.choice(n2, n1, replace=False)] for p in key])
        idx = mods["test_ball_query"].ball_query_np(query, key, r, k, transpose=False)
        out.update({tag + "_query": query, tag + "_key": key, tag + "_idx": idx.astype(np.int64),
                    tag + "_r": np.float64(r), tag + "_k": np.int64(k)})
    np.savez_compressed(os.path.join(HERE, "ball_query.npz"), **out)

    # ---- group_points forward and backward (upstream gradient of ones) ----
    out = {}
    for tag, (b, c, n1, n2, k) in {"a": (2, 3, 512, 128, 32), "b": (2, 8, 65, 33, 7)}.items():
        torch.manual_seed(0)
        f = torch.randn(b, c, n1).requires_grad_(True)
        idx = torch.randint(0, n1, [b, n2, k]).long()
        o = mods["test_group_points"].group_points_builtin(f, idx)
        o.backward(torch.ones_like(o))
        out.update({tag + "_feature": f.detach().numpy(), tag + "_index": idx.numpy(), tag + "_out": o.detach().numpy(),
                    tag + "_grad": f.grad.numpy()})
    np.savez_compressed(os.path.join(HERE, "group_points.npz"), **out)

    # ---- interpolate forward and backward ----
    out = {}
    for tag, (b, c, n1, n2) in {"a": (2, 16, 128, 512), "b": (3, 5, 129, 513)}.items():
        torch.manual_seed(0)
        f = torch.randn(b, c, n1).double().requires_grad_(True)
        idx = torch.randint(0, n1, [b, n2, 3]).long()
        w = torch.rand(b, n2, 3).double()
        w = w / w.sum(dim=2, keepdim=True)
        nb = mods["test_interpolate_feature"].group_points_torch(f, idx)
        o = (nb * w.unsqueeze(1)).sum(dim=-1)
        o.backward(torch.ones_like(o))
        out.update({tag + "_feature": f.detach().numpy(), tag + "_index": idx.numpy(), tag + "_weight": w.numpy(),
                    tag + "_out": o.detach().numpy(), tag + "_grad": f.grad.numpy()})
    np.savez_compressed(os.path.join(HERE, "interpolate.npz"), **out)
    callers()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
