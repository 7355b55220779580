#!/usr/bin/env python
"""Benchmark of the point-cloud neighbour-search hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference|reference-cuda]

Headline workload (config.workload "c4_chamfer_fwd_bwd"): chamfer distance forward + backward on
B=64 cloud pairs of N=M=16384 points (per-cloud mixture of 8 Gaussians, seed 3), batch-sharded over
the N GPUs of one node (one process per GPU, launched by torchrun for N>1), with one scalar loss
all-reduce per step.  One step = one forward + backward over the whole batch.  The metric is
directed point pairs per second (2*B*N*M pairs per step).  Total work is fixed as N grows
("strong" scaling).

The JSON line also carries:
  roofline      the forward kernel (the dominant launch) against the FP32 FMA rate measured live by
                a dependent-FFMA kernel; 8 flop per pair (3 sub, 3 mul, 2 add);
  cpu_baseline  the reference's pure-PyTorch brute-force formulation of the same step, timed on the
                host cores on a bounded sample (rank 0, N=1 only); extras.cpu_baselines holds the
                CPU formulations of the other configurations;
  loss          the global mean chamfer loss of the batch -- the same number for every N;
  e2e           the same metric through the public API with HOST inputs: pinned host -> device
                copies of both clouds and a device -> host read of the loss inside the timed region;
  extras        the other configurations (KNN, FPS / ball query / grouping, 3-NN interpolation).

--impl reference runs the reference's CPU formulation alone (rank 0; other ranks exit), one whole
16384 x 16384 cloud pair per step;
--impl reference-cuda times the reference's own CUDA extension as shipped (default nvcc flags),
when oracle/_ref/shipped/_C.so has been built.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

C4 = dict(B=64, N=16384, M=16384, seed=3)
PAIR_FLOP = 8.0
L2_FLUSH_BYTES = 256 << 20


def env_int(name, default):
    return int(os.environ.get(name, default))


class ClockSampler:
    """nvidia-smi clock / throttle sampling (200 ms) during a timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.idx = device_index
        self.lines = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower() == "active":
                    reasons.add(n)
        if not sm:
            # the sampler produced nothing in time (many ranks starting nvidia-smi at once): one direct query
            try:
                out = subprocess.run(["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-i",
                                      str(self.idx)], capture_output=True, text=True, timeout=20).stdout.strip()
                f = [x.strip() for x in out.split(",")]
                return {"sm_mhz": float(f[1]), "sm_max_mhz": float(f[2]),
                        "reasons": [n for n, v in zip(names, f[5:9]) if v.lower() == "active"], "samples": 1,
                        "note": "single query after the timed region"}
            except Exception:
                return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def flush_l2(buf):
    buf.zero_()


def time_steps(fn, steps, warmup, flush):
    """Per-step CUDA-event timing on the current stream with an L2 flush before each step."""
    for _ in range(warmup):
        flush_l2(flush)
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(steps):
        flush_l2(flush)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        evs.append((s, e))
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in evs]


def rank_max(value, device, world):
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


# ------------------------------------------------------------------------------------------------
def cpu_formulation_rate(sample_rows, repeats=1, threads=None):
    """Reference brute-force PyTorch formulation of chamfer fwd+bwd on the host.

    Sample: the first `sample_rows` points of cloud 0's first cloud against all 16384 points of its
    partner (both directions, forward + autograd backward).  Returns (pairs/s, seconds, pairs)."""
    from oracle import formulations as F
    from torkit3d_b200 import workloads

    torch.set_num_threads(threads or os.cpu_count() or 1)
    x1, x2 = workloads.c4_chamfer_large(num_clouds=1, **{k: C4[k] for k in ("N", "M", "seed")})
    a, b = x1[:, :sample_rows].contiguous(), x2
    pairs = 2.0 * a.size(1) * b.size(1)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        F.chamfer_loss_fwd_bwd(a, b, rows=1024)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return pairs / best, best, pairs


def run_reference_cpu(args, rank, world):
    """The reference's CPU formulation alone: every step is the SAME fixed sample (one whole
    16384 x 16384 cloud pair, forward + backward), so the figure does not depend on a pilot run."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    for _ in range(min(args.warmup, 2)):
        cpu_formulation_rate(C4["N"])
    times = []
    pairs = 0.0
    for _ in range(args.steps):
        _, dt, pairs = cpu_formulation_rate(C4["N"])
        times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = pairs / (ms / 1e3)
    sample = ("CPU formulation (not the reference's CUDA kernels): chamfer fwd+bwd of one whole 16384 x 16384 "
              "cloud pair, both directions, per step")
    line = {"impl": "reference", "metric": "chamfer_point_pairs_per_sec", "value": value, "unit": "pairs/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.gpus, 1),
            "cpu_baseline": {"value": value, "unit": "pairs/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "pairs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def cpu_config_baselines(budget_s=4.0):
    """The reference's brute-force CPU formulations of the other configurations, on the host cores.

    Small configurations run whole; the large ones run a stated sample and the rate is what is
    reported (the sample is named in the result).  Every entry carries its own seconds."""
    import numpy as np

    from oracle import formulations as F
    from torkit3d_b200 import workloads

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    out = {"cores": cores}

    def timed(fn):
        t0 = time.perf_counter()
        fn()
        return time.perf_counter() - t0

    # C1: chamfer fwd+bwd, B=2, 1024 x 1024, whole
    a, b = workloads.c1_chamfer_small()
    F.chamfer_loss_fwd_bwd(a, b)
    dt = min(timed(lambda: F.chamfer_loss_fwd_bwd(a, b)) for _ in range(3))
    out["c1_chamfer_fwd_bwd_ms"] = dt * 1e3
    # C2: KNN k=16 by cdist + topk (torkit3d/ops/native.py), one cloud at a time, 4 of the 16 clouds
    q, r = workloads.c2_knn()
    dt = timed(lambda: [F.knn_cdist_topk(q[i:i + 1], r[i:i + 1], 16) for i in range(4)])
    out["c2_knn_k16_ms"] = dt * 1e3 * 16 / 4
    out["c2_knn_sample"] = "4 of 16 clouds, scaled by 4"
    # C3: FPS (numpy loop of the reference's test), ball query (numpy loop), group (expanded gather)
    p, feat = workloads.c3_set_abstraction()
    pn = p.numpy()
    dt = timed(lambda: F.fps_numpy(pn[:2], 1024))
    out["c3_fps_ms_per_batch"] = dt * 1e3 * 32 / 2
    out["c3_fps_sample"] = "2 of 32 clouds, scaled by 16"
    idx = F.fps_numpy(pn[:1], 1024)
    cent = np.take_along_axis(pn[:1], idx[:, :, None].repeat(3, 2), 1)
    dt = timed(lambda: F.ball_query_numpy(cent[:, :256], pn[:1], 0.1, 32))
    out["c3_ball_query_ms"] = dt * 1e3 * 32 * 4
    out["c3_ball_query_sample"] = "256 of 1024 centroids of 1 of 32 clouds, scaled by 128"
    nbr = torch.from_numpy(F.ball_query_numpy(cent, pn[:1], 0.1, 32)).clamp_(min=0)
    f1 = feat[:1]
    dt = timed(lambda: F.group_gather(f1, nbr))
    out["c3_group_fwd_ms"] = dt * 1e3 * 32
    out["c3_group_fwd_sample"] = "1 of 32 clouds, scaled by 32"
    # C5: three nearest of 32768 keys by cdist + topk, then the weighted gather: 4096 queries of one cloud
    qq, rr, ff = workloads.c5_scene_interp(B=1)
    qs = qq[:, :4096]
    dt = timed(lambda: F.knn_cdist_topk(qs, rr, 3))
    out["c5_three_nn_ms"] = dt * 1e3 * 8 * 131072 / 4096
    d, i = F.knn_cdist_topk(qs, rr, 3)
    w = F.three_nn_weight(d * d)
    dt = timed(lambda: F.interpolate_gather(ff, i, w))
    out["c5_interp_fwd_ms"] = dt * 1e3 * 8 * 131072 / 4096
    out["c5_sample"] = "4096 of 131072 queries of 1 of 8 clouds, scaled by 256"
    return out


def workload_config(n_gpus, world):
    return {"workload": "c4_chamfer_fwd_bwd", "B": C4["B"], "N": C4["N"], "M": C4["M"], "seed": C4["seed"],
            "points": "per-cloud mixture of 8 isotropic Gaussians, sigma 0.1, centres uniform in [-1,1]^3",
            "sharding": "batch over %d GPU(s), scalar loss all-reduce" % n_gpus,
            "l2": "256 MiB buffer written before every timed step (inputs are 25 MB, smaller than L2)"}


# ------------------------------------------------------------------------------------------------
def measure_fp32_peak(lib, dev):
    """Sustained FP32 FMA rate from the library's dependent-chain kernel (TFLOP/s)."""
    sink = torch.zeros(1, device=dev)
    flop = ctypes.c_double(0)
    st = torch.cuda.current_stream().cuda_stream
    iters = 4096
    best = 0.0
    for _ in range(5):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        rc = lib.tk3d_diag_ffma(iters, sink.data_ptr(), ctypes.byref(flop), st)
        e.record()
        torch.cuda.synchronize()
        if rc != 0:
            return None
        best = max(best, flop.value / (s.elapsed_time(e) * 1e-3) / 1e12)
    return best


def extras(dev, rank, world, flush):
    """The other configurations, sharded as they would be in a multi-GPU job."""
    import torch.distributed as dist  # noqa: F401

    from torkit3d_b200 import workloads
    from torkit3d_b200.dist import batch_shard, query_slab
    from torkit3d_b200.ops import (ball_query, group_points, interpolate_feature, knn_points, nn_distance,
                                   sample_farthest_points, three_nn_weight)

    out = {}

    def t(fn, steps=5, warm=3):
        ms = time_steps(fn, steps, warm, flush)
        return rank_max(sum(ms) / len(ms), dev, world)

    # C1 (replicated: too small to shard)
    x1, x2 = [v.to(dev) for v in workloads.c1_chamfer_small()]
    ms = t(lambda: nn_distance(x1, x2), steps=10)
    out["c1_chamfer_fwd_ms"] = ms
    # the same configuration, forward + backward, eager launches against a replayed CUDA graph
    from torkit3d_b200 import _C
    g1 = torch.full((x1.size(0), x1.size(1)), 1e-3, device=dev)
    g2 = torch.full((x2.size(0), x2.size(1)), 1e-3, device=dev)

    def c1_chain():
        d1, i1, d2, i2 = _C.chamfer_distance_forward_cuda(x1, x2)
        return _C.chamfer_distance_backward_cuda(g1, g2, x1, x2, i1, i2)
    out["c1_chamfer_fwd_bwd_eager_ms"] = t(c1_chain, steps=10)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        c1_chain()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        keep = c1_chain()
    out["c1_chamfer_fwd_bwd_graph_ms"] = t(graph.replay, steps=10)
    del graph, keep
    # C2 KNN, batch-sharded
    q, r = workloads.c2_knn()
    q, r = batch_shard(q, rank, world).to(dev), batch_shard(r, rank, world).to(dev)
    ms = t(lambda: knn_points(q, r, 16), steps=10)
    out["c2_knn_k16_ms"] = ms
    out["c2_knn_pairs_per_sec"] = 16 * 4096 * 4096 / (ms * 1e-3)
    # C3 FPS -> ball query -> group, batch-sharded
    p, feat = workloads.c3_set_abstraction()
    p, feat = batch_shard(p, rank, world).to(dev), batch_shard(feat, rank, world).to(dev)
    ms = t(lambda: sample_farthest_points(p, 1024), steps=5)
    out["c3_fps_ms_per_batch"] = ms
    out["c3_fps_evals_per_sec"] = 32 * 1023 * 8192 / (ms * 1e-3)
    idx = sample_farthest_points(p, 1024)
    cent = torch.gather(p, 1, idx.unsqueeze(2).expand(-1, -1, 3)).contiguous()
    ms = t(lambda: ball_query(cent, p, 0.1, 32, transpose=False), steps=10)
    out["c3_ball_query_ms"] = ms
    out["c3_ball_query_pairs_per_sec"] = 32 * 1024 * 8192 / (ms * 1e-3)
    nbr = ball_query(cent, p, 0.1, 32, transpose=False)
    ms = t(lambda: group_points(feat, nbr), steps=10)
    out["c3_group_fwd_ms"] = ms
    out["c3_group_fwd_GBps"] = 343.9e6 / (ms * 1e-3) / 1e9
    featg = feat.clone().requires_grad_(True)
    g = group_points(featg, nbr)
    go = torch.ones_like(g)
    ms = t(lambda: torch.autograd.grad(g, featg, go, retain_graph=True), steps=10)
    out["c3_group_bwd_ms"] = ms
    del g, go, featg
    # C3 as the layer calls it ([B,3,N] layout): fused front ends against the operator chain
    from torkit3d_b200 import _fused
    pcf = p.transpose(1, 2).contiguous()
    ms = t(lambda: _fused.fps_gather(pcf, 1024), steps=5)
    out["c3_fps_gather_fused_ms"] = ms
    _, ccf = _fused.fps_gather(pcf, 1024)
    ms = t(lambda: _fused.sa_group_forward(pcf, ccf, feat, 0.1, 32, want_index=False), steps=10)
    out["c3_sa_group_fused_ms"] = ms

    def sa_chain():
        ii = ball_query(ccf, pcf, 0.1, 32)
        return torch.cat([group_points(feat, ii), group_points(pcf, ii) - ccf.unsqueeze(-1)], dim=1)
    out["c3_sa_group_chain_ms"] = t(sa_chain, steps=10)
    del pcf, ccf
    # C5 three-NN interpolation, query slabs
    qq, rr, ff = workloads.c5_scene_interp()
    qq = query_slab(qq, rank, world).contiguous().to(dev)
    rr, ff = rr.to(dev), ff.to(dev)
    ms = t(lambda: knn_points(qq, rr, 3), steps=3, warm=3)
    out["c5_three_nn_ms"] = ms
    out["c5_three_nn_pairs_per_sec"] = 8 * 131072 * 32768 / (ms * 1e-3)
    d, i = knn_points(qq, rr, 3)
    w = three_nn_weight(d)
    ms = t(lambda: interpolate_feature(ff, i, w), steps=5)
    out["c5_interp_fwd_ms"] = ms
    out["c5_interp_fwd_GBps"] = 708.9e6 / (ms * 1e-3) / 1e9
    # the same gather from features kept as rows (built once per step, shared by all slabs of a scene)
    from torkit3d_b200.ops import feature_rows
    out["c5_feature_rows_ms"] = t(lambda: feature_rows(ff), steps=5)
    frows = feature_rows(ff)
    out["c5_interp_fwd_from_rows_ms"] = t(lambda: interpolate_feature(ff, i, w, rows=frows), steps=5)
    del frows
    ffg = ff.clone().requires_grad_(True)
    o = interpolate_feature(ffg, i, w)
    go = torch.ones_like(o)
    ms = t(lambda: torch.autograd.grad(o, ffg, go, retain_graph=True), steps=5)
    out["c5_interp_bwd_ms"] = ms
    del o, go, ffg
    qcf, rcf = qq.transpose(1, 2).contiguous(), rr.transpose(1, 2).contiguous()
    out["c5_three_nn_interp_fused_ms"] = t(lambda: _fused.three_nn_interp_forward(qcf, rcf, ff), steps=3)
    del qcf, rcf, qq, rr, ff
    # EdgeConv edge features of one DGCNN layer (B=32, 1024 points, C=64, K=20), batch-sharded
    from torkit3d_b200.ops import get_edge_feature
    gen = torch.Generator().manual_seed(7)
    pts = batch_shard(torch.randn(32, 1024, 3, generator=gen), rank, world).to(dev)
    x = batch_shard(torch.randn(32, 64, 1024, generator=gen), rank, world).to(dev)
    _, ind = knn_points(pts, pts, 20)
    ms = t(lambda: get_edge_feature(x, x, ind), steps=10)
    out["edge_feature_fused_ms"] = ms
    out["edge_feature_fused_GBps"] = (32 * 128 * 1024 * 20 * 4 + 32 * 1024 * 20 * 8 + 2 * 32 * 64 * 1024 * 4) / (ms * 1e-3) / 1e9

    def edge_chain():
        grouped = group_points(x, ind)
        xe = x.unsqueeze(3).expand_as(grouped)
        return torch.cat([grouped - xe, xe], dim=1)
    out["edge_feature_chain_ms"] = t(edge_chain, steps=10)
    # DGCNN's feature-space KNN on the same layer (k=20 among 1024 points, 64 channels)
    from torkit3d_b200.ops import knn as feature_knn
    ms = t(lambda: feature_knn(x, x, 20, transpose=True), steps=10)
    out["feature_knn_ms"] = ms
    out["feature_knn_pair_channels_per_sec"] = x.size(0) * 1024 * 1024 * 64 / (ms * 1e-3)
    xt = x.transpose(1, 2)
    out["feature_knn_cdist_topk_ms"] = t(lambda: torch.topk(torch.cdist(xt, xt), 20, dim=2, largest=False), steps=10)
    del x, xt, pts, ind
    # beyond the five configurations: large k (radix selection) and clouds beyond one block (cluster FPS)
    q4, r4 = [batch_shard(v[:8], rank, world).to(dev) for v in workloads.c2_knn()]
    out["knn_k200_ms"] = t(lambda: knn_points(q4, r4, 200), steps=5)
    gen = torch.Generator().manual_seed(9)
    big = batch_shard(torch.rand(8, 65536, 3, generator=gen), rank, world).to(dev)
    out["fps_65536_to_2048_ms"] = t(lambda: sample_farthest_points(big, 2048), steps=3)
    del q4, r4, big
    if world > 1:
        # hardware check of the query-slab sharding: every rank interpolates its slab of a small
        # scene, the slabs are gathered and compared with the unsharded result on every rank
        qs, rs, fs = [v.to(dev) for v in workloads.c5_scene_interp(B=2, NQ=2048 * world, NR=4096, C=16, seed=11)]
        d, i = knn_points(qs, rs, 3)
        whole = interpolate_feature(fs, i, three_nn_weight(d))
        mine_q = query_slab(qs, rank, world).contiguous()
        dm, im = knn_points(mine_q, rs, 3)
        part = interpolate_feature(fs, im, three_nn_weight(dm)).contiguous()
        parts = [torch.empty_like(part) for _ in range(world)]
        idxs = [torch.empty_like(im) for _ in range(world)]
        dist.all_gather(parts, part)
        dist.all_gather(idxs, im)
        out["c5_slabs_equal_unsharded"] = bool(torch.equal(torch.cat(idxs, 1), i)
                                               and torch.allclose(torch.cat(parts, 2), whole, rtol=1e-5, atol=1e-6))
    return out


def run_b200(args, rank, world, local_rank):
    import torch.distributed as dist

    from torkit3d_b200 import _lib, workloads
    from torkit3d_b200.dist import HostCloudPrefetcher, chamfer_loss, chamfer_step, shard_range

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    lib = _lib.load()

    b0, b1 = shard_range(C4["B"], rank, world)
    x1h, x2h = workloads.c4_chamfer_large(first_cloud=b0, num_clouds=b1 - b0, **{k: C4[k] for k in ("B", "N", "M", "seed")})
    x1h, x2h = x1h.pin_memory(), x2h.pin_memory()
    x1 = x1h.to(dev).requires_grad_(True)
    x2 = x2h.to(dev).requires_grad_(True)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    pairs_total = 2.0 * C4["B"] * C4["N"] * C4["M"]
    pairs_local = 2.0 * (b1 - b0) * C4["N"] * C4["M"]

    def step():
        # loss and both gradients in one call; the gradient kernels overlap the scalar all-reduce
        return chamfer_step(x1, x2, global_batch=C4["B"])

    def step_autograd():
        x1.grad = None
        x2.grad = None
        loss = chamfer_loss(x1, x2, global_batch=C4["B"])
        loss.backward()
        return loss

    # ---- device-resident timing: barrier + sync, K steps timed with CUDA events, max over ranks
    barrier(world)
    clk = ClockSampler(local_rank)
    clk.__enter__()  # sampled through every timed region below (value, kernel-only, end-to-end)
    ms = time_steps(step, args.steps, args.warmup, flush)
    barrier(world)
    ms_step = rank_max(sum(ms) / len(ms), dev, world)
    value = pairs_total / (ms_step * 1e-3)
    loss_value = float(step()[0])  # identical on every rank and for every number of GPUs
    ms_auto = time_steps(step_autograd, args.steps, 3, flush)
    ms_step_autograd = rank_max(sum(ms_auto) / len(ms_auto), dev, world)

    # ---- forward kernel alone (the dominant launch), through the C ABI with preallocated outputs
    Bl = b1 - b0
    d1 = torch.empty(Bl, C4["N"], device=dev)
    d2 = torch.empty(Bl, C4["M"], device=dev)
    i1 = torch.empty(Bl, C4["N"], dtype=torch.int64, device=dev)
    i2 = torch.empty(Bl, C4["M"], dtype=torch.int64, device=dev)
    sums = torch.zeros(2, dtype=torch.float64, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    xa, xb = x1.detach(), x2.detach()

    def fwd_only():
        rc = lib.tk3d_chamfer_fwd(xa.data_ptr(), xb.data_ptr(), Bl, C4["N"], C4["M"], d1.data_ptr(), i1.data_ptr(),
                                  d2.data_ptr(), i2.data_ptr(), sums.data_ptr(), 0, st)
        assert rc == 0

    fms = time_steps(fwd_only, args.steps, 3, flush)
    fwd_ms = sum(fms) / len(fms)
    peak = measure_fp32_peak(lib, dev)
    nominal = 148 * 128 * 2 * 1.965e9 / 1e12
    achieved = pairs_local * PAIR_FLOP / (fwd_ms * 1e-3) / 1e12
    fwd_kernel = lib.tk3d_chamfer_fwd_kernel_name(Bl, C4["N"], C4["M"], 0).decode()
    roofline = {"bound": "fp32", "kernel": fwd_kernel, "achieved": achieved,
                "peak": peak if peak else nominal, "peak_source": "measured live (dependent FFMA chains)" if peak
                else "nominal 148 SM x 128 lanes x 2 x 1.965 GHz", "unit": "TFLOP/s",
                "frac": achieved / (peak if peak else nominal), "nominal_peak": nominal,
                "frac_nominal": achieved / nominal,
                # DRAM read + write per launch: an ncu capture of this kernel on 24 cloud pairs moved
                # 9.465 MB (the clouds themselves, read once); scaled by the clouds of this launch
                "traffic": 9.465e6 * Bl / 24.0, "traffic_unit": "bytes",
                "traffic_source": "ncu capture at 24 cloud pairs, scaled by cloud count",
                "flop_per_pair": PAIR_FLOP, "pairs_per_launch": pairs_local, "launch_ms": fwd_ms,
                "pairs_per_sec": pairs_local / (fwd_ms * 1e-3)}

    # ---- backward kernels alone (HBM-bound)
    g1 = torch.full((Bl, C4["N"]), 1e-6, device=dev)
    g2 = torch.full((Bl, C4["M"]), 1e-6, device=dev)
    ga = torch.empty(Bl, C4["N"], 3, device=dev)
    gb = torch.empty(Bl, C4["M"], 3, device=dev)

    def bwd_only():
        rc = lib.tk3d_chamfer_bwd(g1.data_ptr(), g2.data_ptr(), xa.data_ptr(), xb.data_ptr(), i1.data_ptr(),
                                  i2.data_ptr(), Bl, C4["N"], C4["M"], ga.data_ptr(), gb.data_ptr(), 0, st)
        assert rc == 0

    bms = time_steps(bwd_only, args.steps, 3, flush)
    bwd_ms = sum(bms) / len(bms)
    bwd_bytes = Bl * (C4["N"] + C4["M"]) * (2 * 12 + 8 + 4)
    hbm_peak = None
    try:
        hbm_peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
    except (OSError, KeyError, ValueError):
        hbm_peak = 6650.0
    bwd = {"bound": "hbm", "kernels": "chamfer_bwd_own_kernel + chamfer_bwd_scatter_kernel", "launch_ms": bwd_ms,
           "achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
           "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / hbm_peak, "bytes": bwd_bytes}

    # ---- end to end: host inputs in pinned memory, H2D inside the timed region, loss read back
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    pf = HostCloudPrefetcher(dev)
    step_ws = {}  # output tensors of the step, reused from step to step

    def e2e_run(steps):
        # every step's clouds come from pinned host memory; the copy of step i+1 is enqueued on a
        # side stream before the kernels of step i (double buffering), the loss is read back and
        # the host waits for it every step
        pf.prefetch(x1h, x2h)
        for i in range(steps):
            a, b = pf.get()
            loss, _, _ = chamfer_step(a, b, global_batch=C4["B"], workspace=step_ws)
            if i + 1 < steps:
                pf.prefetch(x1h, x2h)  # behind this step's launches; its copy still overlaps them
            loss_host.copy_(loss, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        return float(loss_host)

    e2e_run(max(3, args.warmup))
    barrier(world)
    t0 = time.perf_counter()
    e2e_run(args.steps)  # K copies, K forward+backward steps and K read-backs inside the timed region
    barrier(world)
    e2e_s = rank_max(time.perf_counter() - t0, dev, world) / args.steps
    clk.__exit__(None, None, None)
    clocks = clk.summary()
    e2e = {"value": pairs_total / e2e_s, "unit": "pairs/s", "ms_per_step": e2e_s * 1e3,
           "h2d_bytes_per_step": int(x1h.numel() * 4 + x2h.numel() * 4), "d2h_bytes_per_step": 4,
           "api": "HostCloudPrefetcher (pinned host clouds, next step's copy on a side stream) + "
                  "dist.chamfer_step (loss + gradients), loss read back every step"}

    ext = extras(dev, rank, world, flush) if not args.no_extras else {}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        # about 10-20 s of host work: whole cloud pairs (16384 x 16384, both directions), repeated
        t_total, pairs_total_cpu, reps = 0.0, 0.0, 0
        while t_total < 10.0 and reps < 64:
            _, dt, pairs = cpu_formulation_rate(C4["N"])
            t_total += dt
            pairs_total_cpu += pairs
            reps += 1
        cpu = {"value": pairs_total_cpu / t_total, "unit": "pairs/s", "cores": cores, "kind": "port",
               "seconds": t_total,
               "sample": "reference brute-force PyTorch formulation (difference tensor in 1024-row blocks, min, "
                         "autograd backward) of chamfer fwd+bwd on one 16384 x 16384 cloud pair, repeated %d times" % reps}

        if not args.no_extras:
            ext["cpu_baselines"] = cpu_config_baselines()

    if rank == 0:
        line = {"metric": "chamfer_point_pairs_per_sec", "value": value, "unit": "pairs/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(world, world), "clocks": clocks, "e2e": e2e, "gpu_launches": 4,
                "gpu_launches_detail": "per step: %s, chamfer_bwd_own_kernel, chamfer_bwd_scatter_kernel, chamfer_mean_loss_kernel" % roofline["kernel"],
                "loss": loss_value, "ms_per_step_autograd": ms_step_autograd,
                "roofline": roofline, "roofline_backward": bwd, "cpu_baseline": cpu, "extras": ext}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()


def run_reference_cuda(args, rank, world, local_rank):
    """The reference's own CUDA extension as shipped (default nvcc flags), same step, 1 GPU."""
    import importlib.util

    if rank != 0:
        return
    so = os.path.join(ROOT, "oracle", "_ref", "shipped", "_C.so")
    if not (os.path.exists(so) and torch.cuda.is_available()):
        print(json.dumps({"impl": "reference-cuda", "unavailable": "oracle/_ref/shipped/_C.so not built or no GPU"}))
        return
    from torkit3d_b200 import workloads

    spec = importlib.util.spec_from_file_location("_C", so)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    dev = torch.device("cuda", 0)
    x1, x2 = [v.to(dev) for v in workloads.c4_chamfer_large(**C4)]
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    g1 = torch.full((C4["B"], C4["N"]), 1e-6, device=dev)
    g2 = torch.full((C4["B"], C4["M"]), 1e-6, device=dev)

    def step():
        d1, i1, d2, i2 = ref.chamfer_distance_forward_cuda(x1, x2)
        (d1.mean() + d2.mean())
        ref.chamfer_distance_backward_cuda(g1, g2, x1, x2, i1, i2)

    ms = time_steps(step, args.steps, args.warmup, flush)
    ms_step = sum(ms) / len(ms)
    pairs = 2.0 * C4["B"] * C4["N"] * C4["M"]
    ext = {}
    if not args.no_extras:
        def t(fn, steps=3):
            v = time_steps(fn, steps, 2, flush)
            return sum(v) / len(v)

        d1, i1, d2, i2 = ref.chamfer_distance_forward_cuda(x1, x2)
        ext["c4_chamfer_fwd_ms"] = t(lambda: ref.chamfer_distance_forward_cuda(x1, x2))
        ext["c4_chamfer_bwd_ms"] = t(lambda: ref.chamfer_distance_backward_cuda(g1, g2, x1, x2, i1, i2))
        del x1, x2, d1, i1, d2, i2
        q, r = [v.to(dev) for v in workloads.c2_knn()]
        ext["c2_knn_k16_ms"] = t(lambda: ref.knn_distance_cuda(q, r, 16, 1))
        p, feat = [v.to(dev) for v in workloads.c3_set_abstraction()]
        ext["c3_fps_ms_per_batch"] = t(lambda: ref.sample_farthest_points_cuda(p, 1024))
        idx = ref.sample_farthest_points_cuda(p, 1024)
        cent = torch.gather(p, 1, idx.unsqueeze(2).expand(-1, -1, 3)).contiguous()
        ext["c3_ball_query_ms"] = t(lambda: ref.ball_query_cuda(cent, p, 0.1, 32))
        nbr = ref.ball_query_cuda(cent, p, 0.1, 32)
        ext["c3_group_fwd_ms"] = t(lambda: ref.group_points_forward_cuda(feat, nbr))
        go = torch.ones(32, 64, 1024, 32, device=dev)
        ext["c3_group_bwd_ms"] = t(lambda: ref.group_points_backward_cuda(go, nbr, 8192))
        del go
        qq, rr, ff = [v.to(dev) for v in workloads.c5_scene_interp()]
        ext["c5_three_nn_ms"] = t(lambda: ref.knn_distance_cuda(qq, rr, 3, 1), steps=2)
        d, i = ref.knn_distance_cuda(qq, rr, 3, 1)
        inv = 1.0 / torch.clamp(d, min=1e-10)
        w = inv / inv.sum(2, keepdim=True)
        ext["c5_interp_fwd_ms"] = t(lambda: ref.interpolate_forward_cuda(ff, i, w))
    print(json.dumps({"impl": "reference-cuda", "metric": "chamfer_point_pairs_per_sec", "value": pairs / (ms_step * 1e-3),
                      "unit": "pairs/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                      "higher_is_better": True, "dtype": "f32", "data": "synthetic", "config": workload_config(1, 1),
                      "extras": ext,
                      "note": "reference torkit3d._C compiled unmodified for sm_100a with default nvcc flags"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-cuda"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    world = env_int("WORLD_SIZE", 1)
    rank = env_int("RANK", 0)
    local_rank = env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference_cpu(args, rank, world)
        return
    if args.impl == "reference-cuda":
        run_reference_cuda(args, rank, world, local_rank)
        return
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_b200(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
