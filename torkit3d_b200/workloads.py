"""Seeded synthetic inputs for the five benchmark configurations.

The reference measures on no public dataset; these generators stand in for real point clouds.
Everything is drawn in fp32 on the CPU from ``torch.Generator().manual_seed(seed)`` so that the CPU
oracle and every GPU see identical bits.  ``scale`` shrinks the batch / point counts for tests
(1.0 = the full configuration).
"""
import torch


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def c1_chamfer_small(B=2, N=1024, M=1024, seed=0):
    """Chamfer fwd+bwd, points i.i.d. uniform in [-1,1]^3."""
    g = _gen(seed)
    xyz1 = torch.rand(B, N, 3, generator=g) * 2 - 1
    xyz2 = torch.rand(B, M, 3, generator=g) * 2 - 1
    return xyz1, xyz2


def c2_knn(B=16, N1=4096, N2=4096, seed=1):
    """KNN distance+index, query/key ~ N(0, I3); k=16 in the full configuration."""
    g = _gen(seed)
    query = torch.randn(B, N1, 3, generator=g)
    key = torch.randn(B, N2, 3, generator=g)
    return query, key


def c3_set_abstraction(B=32, N=8192, C=64, seed=2):
    """Unit-sphere surface samples + N(0, 0.01^2) jitter, and [B,C,N] features ~ N(0,1).

    Full configuration: FPS 8192 -> 1024 from index 0, ball_query r=0.1 K=32, group_points.
    """
    g = _gen(seed)
    p = torch.randn(B, N, 3, generator=g)
    p = p / p.norm(dim=2, keepdim=True)
    p = p + 0.01 * torch.randn(B, N, 3, generator=g)
    feat = torch.randn(B, C, N, generator=g)
    return p.contiguous(), feat


def c4_chamfer_large(B=64, N=16384, M=16384, seed=3, first_cloud=0, num_clouds=None):
    """Per-cloud mixture of 8 isotropic Gaussians (centres uniform in [-1,1]^3, sigma 0.1).

    Both clouds of a pair share the same 8 centres.  Each cloud pair is drawn from its own
    generator (seed * 1000003 + cloud index) so that a batch shard ``[first_cloud, first_cloud +
    num_clouds)`` holds exactly the clouds the unsharded batch holds at those positions.
    """
    if num_clouds is None:
        num_clouds = B - first_cloud
    xs, ys = [], []
    for c in range(first_cloud, first_cloud + num_clouds):
        g = _gen(seed * 1000003 + c)
        centres = torch.rand(8, 3, generator=g) * 2 - 1
        a = centres[torch.randint(0, 8, (N,), generator=g)] + 0.1 * torch.randn(N, 3, generator=g)
        b = centres[torch.randint(0, 8, (M,), generator=g)] + 0.1 * torch.randn(M, 3, generator=g)
        xs.append(a)
        ys.append(b)
    return torch.stack(xs).contiguous(), torch.stack(ys).contiguous()


def c5_scene_interp(B=8, NQ=131072, NR=32768, C=128, seed=4):
    """Query / reference points uniform in a 10 x 10 x 3 m box and [B,C,NR] features ~ N(0,1)."""
    g = _gen(seed)
    box = torch.tensor([10.0, 10.0, 3.0])
    q = torch.rand(B, NQ, 3, generator=g) * box
    r = torch.rand(B, NR, 3, generator=g) * box
    feat = torch.randn(B, C, NR, generator=g)
    return q.contiguous(), r.contiguous(), feat
