"""World-size-2 `gloo` tests (CPU) of the multi-GPU host logic: shard arithmetic, and the sharded
chamfer loss with its single scalar all-reduce.  The CUDA kernels are replaced by the CPU oracle
through the helper's test hooks; everything else (partial sums, all-reduce, gradient scaling) is the
code that runs on the GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from torkit3d_b200.dist import batch_shard, query_slab, shard_range


def test_shard_ranges_tile_the_batch():
    for total in (0, 1, 7, 8, 64, 131072):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a1 >= a0
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)
    t = torch.arange(2 * 10 * 3).view(2, 10, 3)
    assert torch.equal(torch.cat([query_slab(t, r, 4) for r in range(4)], 1), t)
    assert torch.equal(torch.cat([batch_shard(t, r, 2) for r in range(2)], 0), t)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_forward(a, b, sums):
    from oracle import oracle as orc

    d1, i1, d2, i2 = orc.chamfer_fwd(a.detach().numpy(), b.detach().numpy(), threads=1)
    sums[0] = float(d1.astype(np.float64).sum())
    sums[1] = float(d2.astype(np.float64).sum())
    return torch.from_numpy(d1), torch.from_numpy(i1), torch.from_numpy(d2), torch.from_numpy(i2)


def _oracle_backward(g1, g2, a, b, i1, i2):
    from oracle import oracle as orc

    ga, gb = orc.chamfer_bwd(g1.numpy(), g2.numpy(), a.detach().numpy(), b.detach().numpy(), i1.numpy(), i2.numpy(),
                             threads=1)
    return torch.from_numpy(ga), torch.from_numpy(gb)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torkit3d_b200 import workloads
        from torkit3d_b200.dist import chamfer_loss

        B, N, M = 6, 200, 150
        b0, b1 = shard_range(B, rank, world)
        x1, x2 = workloads.c4_chamfer_large(B=B, N=N, M=M, first_cloud=b0, num_clouds=b1 - b0)
        x1.requires_grad_(True)
        x2.requires_grad_(True)
        loss = chamfer_loss(x1, x2, global_batch=B, _forward_fn=_oracle_forward, _backward_fn=_oracle_backward)
        loss.backward()
        torch.save({"loss": loss.detach(), "g1": x1.grad, "g2": x2.grad, "range": (b0, b1)},
                   os.path.join(out_dir, "rank%d.pt" % rank))
    finally:
        dist.destroy_process_group()


def test_sharded_chamfer_loss_world2(tmp_path, oracle):
    from torkit3d_b200 import workloads
    from torkit3d_b200.dist import chamfer_loss

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / ("rank%d.pt" % r)) for r in range(world)]
    # single-process result over the whole batch
    B, N, M = 6, 200, 150
    x1, x2 = workloads.c4_chamfer_large(B=B, N=N, M=M)
    x1.requires_grad_(True)
    x2.requires_grad_(True)
    loss = chamfer_loss(x1, x2, _forward_fn=_oracle_forward, _backward_fn=_oracle_backward)
    loss.backward()
    # independent statement of the loss
    d1, _, d2, _ = oracle.chamfer_fwd(x1.detach().numpy(), x2.detach().numpy())
    np.testing.assert_allclose(float(loss), d1.mean(dtype=np.float64) + d2.mean(dtype=np.float64), rtol=1e-6)
    for p in parts:
        np.testing.assert_allclose(float(p["loss"]), float(loss), rtol=1e-6)  # identical on every rank
        b0, b1 = p["range"]
        torch.testing.assert_close(p["g1"], x1.grad[b0:b1], rtol=1e-6, atol=1e-9)
        torch.testing.assert_close(p["g2"], x2.grad[b0:b1], rtol=1e-6, atol=1e-9)
    assert [p["range"] for p in parts] == [(0, 3), (3, 6)]
