"""Run one operator on one benchmark configuration a few times (for profilers and quick timings).

    python run_case.py <case> [--iters 3] [--scale-batch B]

Cases: c1_chamfer, c2_knn, c3_fps, c3_ball, c3_group_fwd, c3_group_bwd, c4_chamfer_fwd,
c4_chamfer_bwd, c5_three_nn, c5_three_nn_slab8, c5_interp_fwd, c5_interp_fwd_rows, c5_feature_rows, c5_interp_bwd, and the layer front ends on the same
inputs in channel-first layout, fused and spelled operator by operator: c3_fps_gather,
c3_fps_chain, c3_sa_fused, c3_sa_chain, c3_sa_fused_bwd, c5_fp_fused, c5_fp_chain; and the EdgeConv edge
features of a DGCNN layer (B=32, 1024 points, C=64, K=20): edge_fused, edge_chain; and its feature-space
KNN: feature_knn, feature_knn_chain (cdist + topk in PyTorch); knn_f64 (float64 KNN, 8 x 2048 x 2048, k=16); knn_k200 (float32, 4 x 4096 x 4096, k=200); fps_large (4 clouds of 65536 points -> 2048 samples).  ``--scale-batch`` overrides the batch
size of the configuration (smaller captures for ``ncu``).  Prints the mean CUDA-event time.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from torkit3d_b200 import _C, workloads  # noqa: E402
from torkit3d_b200.ops import ball_query, knn_points, sample_farthest_points, three_nn_weight  # noqa: E402


def build_case(name, batch, dev):
    kw = {} if batch is None else {"B": batch}
    if name == "c1_chamfer":
        a, b = [t.to(dev) for t in workloads.c1_chamfer_small(**kw)]
        return lambda: _C.chamfer_distance_forward_cuda(a, b)
    if name == "c2_knn":
        q, r = [t.to(dev) for t in workloads.c2_knn(**kw)]
        return lambda: knn_points(q, r, 16)
    if name == "fps_large":
        # clouds beyond one block's registers: 4 clouds of 65536 points -> 2048 samples (a cluster of 8 blocks each)
        g = torch.Generator().manual_seed(9)
        p = torch.rand(batch or 4, 65536, 3, generator=g).to(dev)
        return lambda: sample_farthest_points(p, 2048)
    if name == "knn_k200":
        # large k: the second configuration's clouds (4096 x 4096 per cloud), 4 of them, k=200
        q, r = [t[:(batch or 4)].contiguous().to(dev) for t in workloads.c2_knn()]
        return lambda: knn_points(q, r, 200)
    if name == "knn_f64":
        # float64 clouds with few queries: 8 clouds of 2048 points against 2048 keys, k=16
        B = batch or 8
        g = torch.Generator().manual_seed(8)
        q = torch.randn(B, 2048, 3, generator=g, dtype=torch.float64).to(dev)
        r = torch.randn(B, 2048, 3, generator=g, dtype=torch.float64).to(dev)
        return lambda: knn_points(q, r, 16)
    if name.startswith("feature_knn"):
        # DGCNN's dynamic graph on 64-channel features: B=32 clouds of 1024 points, k=20
        from torkit3d_b200.ops import knn

        B = batch or 32
        g = torch.Generator().manual_seed(9)
        x = torch.randn(B, 64, 1024, generator=g).to(dev)
        if name == "feature_knn":
            return lambda: knn(x, x, 20, transpose=True)

        def knn_chain():  # the reference's formulation on the same GPU
            xt = x.transpose(1, 2)
            return torch.topk(torch.cdist(xt, xt), 20, dim=2, largest=False, sorted=False)
        return knn_chain
    if name.startswith("edge"):
        from torkit3d_b200.ops import get_edge_feature, group_points

        B = batch or 32
        g = torch.Generator().manual_seed(7)
        pts = torch.randn(B, 1024, 3, generator=g).to(dev)
        x = torch.randn(B, 64, 1024, generator=g).to(dev)
        _, ind = knn_points(pts, pts, 20)
        if name == "edge_fused":
            return lambda: get_edge_feature(x, x, ind)

        def edge_chain():
            grouped = group_points(x, ind)
            xe = x.unsqueeze(3).expand_as(grouped)
            return torch.cat([grouped - xe, xe], dim=1)
        return edge_chain
    if name.startswith("c3"):
        p, feat = [t.to(dev) for t in workloads.c3_set_abstraction(**kw)]
        if name == "c3_fps":
            return lambda: sample_farthest_points(p, 1024)
        if name in ("c3_fps_gather", "c3_fps_chain", "c3_sa_fused", "c3_sa_chain", "c3_sa_fused_bwd"):
            from torkit3d_b200 import _fused
            from torkit3d_b200.layers import set_abstraction_group
            from torkit3d_b200.ops import group_points

            pcf = p.transpose(1, 2).contiguous()  # [B,3,N], the layout the reference's layers pass around
            if name == "c3_fps_gather":
                return lambda: _fused.fps_gather(pcf, 1024)
            if name == "c3_fps_chain":
                def fps_chain():
                    i = sample_farthest_points(pcf, 1024, True)
                    return torch.gather(pcf, 2, i.unsqueeze(1).expand(-1, 3, -1))
                return fps_chain
            _, ccf = _fused.fps_gather(pcf, 1024)
            if name == "c3_sa_fused":
                return lambda: _fused.sa_group_forward(pcf, ccf, feat, 0.1, 32, want_index=False)
            if name == "c3_sa_fused_bwd":
                out, i32 = _fused.sa_group_forward(pcf, ccf, feat, 0.1, 32)
                go = torch.randn_like(out)
                return lambda: _fused.sa_group_backward(go, i32, feat.size(1), feat.size(2))

            def sa_chain():
                i = ball_query(ccf, pcf, 0.1, 32)
                return torch.cat([group_points(feat, i), group_points(pcf, i) - ccf.unsqueeze(-1)], dim=1)
            return sa_chain
        idx = sample_farthest_points(p, 1024)
        cent = torch.gather(p, 1, idx.unsqueeze(2).expand(-1, -1, 3)).contiguous()
        if name == "c3_ball":
            return lambda: ball_query(cent, p, 0.1, 32, transpose=False)
        nbr = ball_query(cent, p, 0.1, 32, transpose=False)
        if name == "c3_group_fwd":
            return lambda: _C.group_points_forward_cuda(feat, nbr)
        if name == "c3_group_bwd":
            go = torch.randn(feat.size(0), feat.size(1), 1024, 32, device=dev)
            return lambda: _C.group_points_backward_cuda(go, nbr, feat.size(2))
    if name.startswith("c4"):
        if batch is not None:
            a, b = [t.to(dev) for t in workloads.c4_chamfer_large(num_clouds=batch)]
        else:
            a, b = [t.to(dev) for t in workloads.c4_chamfer_large()]
        if name == "c4_chamfer_fwd":
            return lambda: _C.chamfer_distance_forward_cuda(a, b)
        d1, i1, d2, i2 = _C.chamfer_distance_forward_cuda(a, b)
        g1, g2 = torch.full_like(d1, 1e-6), torch.full_like(d2, 1e-6)
        if name == "c4_chamfer_bwd":
            return lambda: _C.chamfer_distance_backward_cuda(g1, g2, a, b, i1, i2)
    if name.startswith("c5"):
        q, r, feat = [t.to(dev) for t in workloads.c5_scene_interp(**kw)]
        if name in ("c5_fp_fused", "c5_fp_chain"):
            from torkit3d_b200 import _fused
            from torkit3d_b200.ops import interpolate_feature

            qcf, rcf = q.transpose(1, 2).contiguous(), r.transpose(1, 2).contiguous()
            if name == "c5_fp_fused":
                return lambda: _fused.three_nn_interp_forward(qcf, rcf, feat)

            def fp_chain():
                d, i = knn_points(qcf, rcf, 3, transpose=True)
                inv = 1.0 / torch.clamp(d, min=1e-10)
                w = inv / torch.sum(inv, dim=2, keepdim=True)
                return interpolate_feature(feat, i, w)
            return fp_chain
        if name == "c5_three_nn":
            return lambda: knn_points(q, r, 3)
        if name == "c5_three_nn_slab8":  # one rank's query slab of an 8-GPU run, keys replicated
            qs = q[:, :q.size(1) // 8].contiguous()
            return lambda: knn_points(qs, r, 3)
        d, i = knn_points(q, r, 3)
        w = three_nn_weight(d)
        if name == "c5_interp_fwd":
            return lambda: _C.interpolate_forward_cuda(feat, i, w)
        if name == "c5_interp_fwd_rows":
            rows = _C.feature_rows(feat)
            return lambda: _C.interpolate_forward_rows_cuda(rows, i, w)
        if name == "c5_feature_rows":
            return lambda: _C.feature_rows(feat)
        if name == "c5_interp_bwd":
            go = torch.randn(feat.size(0), feat.size(1), q.size(1), device=dev)
            return lambda: _C.interpolate_backward_cuda(go, i, w, feat.size(2))
    raise SystemExit("unknown case " + name)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--scale-batch", type=int, default=None)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    fn = build_case(a.case, a.scale_batch, dev)
    fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    print("%s: %.4f ms per call (%d calls)" % (a.case, s.elapsed_time(e) / a.iters, a.iters))


if __name__ == "__main__":
    main()
