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

    return mods, native_knn


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
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
