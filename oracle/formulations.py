"""TEST INFRASTRUCTURE ONLY -- the reference's brute-force PyTorch / numpy formulations, restated.

The reference has no CPU implementation of its operators; what it does have are the dense
formulations its own tests compare the CUDA ops against.  They are restated here (not imported: the
reference checkout is not present where the benchmark runs) and serve two purposes:

  * a second, independent statement of each operator to cross-check the C oracle;
  * the timed CPU baseline ("the reference's pure-PyTorch brute-force formulation").

Sources restated: tests/ops/test_chamfer_distance.py:8-31 (pairwise difference tensor, min over
each axis), torkit3d/ops/native.py:28-29 (cdist + topk), tests/ops/test_sample_farthest_points.py:
7-38, tests/ops/test_ball_query.py:15-40, tests/ops/test_group_points.py:6-12,
tests/ops/test_interpolate_feature.py:15-22, torkit3d/layers/pointnet2.py:128-130.
"""
import numpy as np
import torch


def pairwise_sqdist(a, b):
    """[B,N,3] x [B,M,3] -> [B,N,M] by materialising the difference tensor."""
    diff = a.unsqueeze(2) - b.unsqueeze(1)
    return (diff ** 2).sum(dim=3)


def chamfer_dense(xyz1, xyz2):
    """(dist1, idx1, dist2, idx2) from the full distance matrix."""
    d = pairwise_sqdist(xyz1, xyz2)
    dist1, idx1 = d.min(dim=2)
    dist2, idx2 = d.min(dim=1)
    return dist1, idx1, dist2, idx2


def chamfer_dense_chunked(xyz1, xyz2, rows=2048):
    """Same result, evaluated in row blocks so the [N,M,3] tensor stays small."""
    B, N, _ = xyz1.shape
    M = xyz2.shape[1]
    dist1 = xyz1.new_empty(B, N)
    idx1 = torch.empty(B, N, dtype=torch.long)
    dist2 = xyz1.new_full((B, M), float("inf"))
    idx2 = torch.zeros(B, M, dtype=torch.long)
    for s in range(0, N, rows):
        d = pairwise_sqdist(xyz1[:, s:s + rows], xyz2)
        dist1[:, s:s + rows], idx1[:, s:s + rows] = d.min(dim=2)
        cd, ci = d.min(dim=1)
        better = cd < dist2
        dist2 = torch.where(better, cd, dist2)
        idx2 = torch.where(better, ci + s, idx2)
    return dist1, idx1, dist2, idx2


def chamfer_loss_fwd_bwd(xyz1, xyz2, rows=2048):
    """mean(dist1)+mean(dist2) and its gradients by autograd through the dense formulation."""
    xyz1 = xyz1.detach().clone().requires_grad_(True)
    xyz2 = xyz2.detach().clone().requires_grad_(True)
    B, N, _ = xyz1.shape
    M = xyz2.shape[1]
    if N * M * B <= 2048 * 16384:
        d = pairwise_sqdist(xyz1, xyz2)
        loss = d.min(dim=2)[0].mean() + d.min(dim=1)[0].mean()
        loss.backward()
        return loss.detach(), xyz1.grad, xyz2.grad
    # Large clouds: indices from the chunked pass, then the loss from gathered pairs.
    with torch.no_grad():
        _, idx1, _, idx2 = chamfer_dense_chunked(xyz1, xyz2, rows)
    nn1 = torch.gather(xyz2, 1, idx1.unsqueeze(2).expand(-1, -1, 3))
    nn2 = torch.gather(xyz1, 1, idx2.unsqueeze(2).expand(-1, -1, 3))
    loss = ((xyz1 - nn1) ** 2).sum(2).mean() + ((xyz2 - nn2) ** 2).sum(2).mean()
    loss.backward()
    return loss.detach(), xyz1.grad, xyz2.grad


def knn_cdist_topk(query, key, k, sorted=True):
    """Euclidean (not squared) distances and indices, as torkit3d.ops.native.knn returns them."""
    d = torch.cdist(query, key)
    return torch.topk(d, k, dim=2, largest=False, sorted=sorted)


def knn_dense_sq(query, key, k):
    """Squared distances from the difference tensor + topk (exact arithmetic, unlike cdist)."""
    d = pairwise_sqdist(query, key)
    return torch.topk(d, k, dim=2, largest=False, sorted=True)


def fps_numpy(points, num_samples):
    """points [B,N,3] numpy -> [B,S] int64; argmax of the running minimum distance."""
    out = np.zeros((points.shape[0], num_samples), np.int64)
    for b, cloud in enumerate(points):
        running = None
        cur = 0
        for s in range(1, num_samples):
            d = np.square(cloud - cloud[cur][None, :]).sum(1)
            running = d if running is None else np.minimum(d, running)
            cur = int(np.argmax(running))
            out[b, s] = cur
    return out


def ball_query_numpy(query, key, radius, k):
    """query [B,N1,3], key [B,N2,3] numpy -> [B,N1,k] int64 (rows without a hit stay -1)."""
    B, N1, _ = query.shape
    out = np.full((B, N1, k), -1, np.int64)
    for b in range(B):
        for i in range(N1):
            d = np.square(key[b] - query[b, i][None, :]).sum(1)
            hit = np.nonzero(d < radius ** 2)[0]
            if hit.size == 0:
                continue
            if hit.size < k:
                out[b, i, :hit.size] = hit
                out[b, i, hit.size:] = hit[0]
            else:
                out[b, i] = hit[:k]
    return out


def group_gather(feature, index):
    b, c, n1 = feature.shape
    _, n2, k = index.shape
    return torch.gather(feature.unsqueeze(2).expand(b, c, n2, n1), 3, index.unsqueeze(1).expand(b, c, n2, k))


def interpolate_gather(feature, index, weight):
    return (group_gather(feature, index) * weight.unsqueeze(1)).sum(dim=-1)


def three_nn_weight(dist):
    inv = 1.0 / torch.clamp(dist, min=1e-10)
    return inv / inv.sum(dim=2, keepdim=True)
