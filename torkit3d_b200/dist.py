"""Multi-GPU use of the operators: one process per GPU, independent shards, one scalar exchange.

Every operator of this package is independent per cloud (batch entry) and -- except farthest point
sampling -- per query point, so a job scales by giving each rank a slice of the batch
(``batch_shard``) or, for a single huge scene, a slab of the query points (``query_slab``) with the
key cloud and its features replicated.  No operator needs another rank's data.  The only exchange
is the scalar chamfer loss: ``chamfer_loss`` produces the local partial sums inside the forward
kernel's epilogue and all-reduces two float64 numbers (NCCL over NVLink when the tensors are on
GPUs; any ``torch.distributed`` backend works, which is how the CPU ``gloo`` tests exercise the
host logic with a stand-in for the kernels).
"""
import torch
import torch.distributed as dist

from .ops._functions import _C


def shard_range(total: int, rank: int, world: int):
    """Contiguous, balanced [begin, end) of ``total`` units for ``rank`` of ``world`` (remainder
    spread over the first ranks).  The ranges of all ranks tile [0, total) in rank order."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank %d / world %d" % (rank, world))
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def batch_shard(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's clouds of a [B, ...] tensor."""
    b, e = shard_range(t.size(0), rank, world)
    return t[b:e]


def query_slab(t: torch.Tensor, rank: int, world: int, dim: int = 1) -> torch.Tensor:
    """This rank's slab of query points along ``dim`` (every cloud keeps all its key points)."""
    b, e = shard_range(t.size(dim), rank, world)
    return t.narrow(dim, b, e - b)


def _world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group)
    return 1


class _ChamferLoss(torch.autograd.Function):
    """loss = sum(dist1)/count1 + sum(dist2)/count2 over ALL ranks' clouds.

    forward: chamfer kernel with fused partial sums -> all-reduce(SUM) of [sum1, sum2] (float64);
    backward: the loss is linear in the distances, so d loss / d dist is the constant 1/count and
    the gradient kernels need no communication.
    """

    @staticmethod
    def forward(ctx, xyz1, xyz2, count1, count2, group, forward_fn, backward_fn):
        a, b = xyz1.contiguous(), xyz2.contiguous()
        sums = torch.zeros(2, dtype=torch.float64, device=a.device)
        _, idx1, _, idx2 = forward_fn(a, b, sums)
        if _world(group) > 1:
            dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
        ctx.save_for_backward(a, b, idx1, idx2)
        ctx.counts = (count1, count2)
        ctx.backward_fn = backward_fn
        loss = sums[0] / count1 + sums[1] / count2
        return loss.to(a.dtype)

    @staticmethod
    def backward(ctx, grad_loss):
        a, b, idx1, idx2 = ctx.saved_tensors
        c1, c2 = ctx.counts
        g1 = (grad_loss.to(a.dtype) / c1).expand(a.size(0), a.size(1)).contiguous()
        g2 = (grad_loss.to(a.dtype) / c2).expand(b.size(0), b.size(1)).contiguous()
        ga, gb = ctx.backward_fn(g1, g2, a, b, idx1, idx2)
        return ga, gb, None, None, None, None, None


def _cuda_forward(a, b, sums):
    return _C.chamfer_distance_forward_cuda(a, b, sums=sums)


def chamfer_loss(xyz1, xyz2, global_batch=None, group=None, _forward_fn=None, _backward_fn=None):
    """Mean chamfer loss ``mean(dist1) + mean(dist2)`` over a batch that is sharded across ranks.

    Args:
        xyz1: [B_local, N1, 3] this rank's clouds.   xyz2: [B_local, N2, 3].
        global_batch: number of clouds over all ranks (default: B_local * world size).
        group: process group (default: the world).

    Returns a scalar, identical on every rank, differentiable w.r.t. both local clouds; the
    gradients are those of the GLOBAL mean.  ``_forward_fn`` / ``_backward_fn`` replace the CUDA
    kernels in host-logic tests.
    """
    world = _world(group)
    gb = int(global_batch) if global_batch is not None else xyz1.size(0) * world
    count1 = float(gb * xyz1.size(1))
    count2 = float(gb * xyz2.size(1))
    return _ChamferLoss.apply(xyz1, xyz2, count1, count2, group, _forward_fn or _cuda_forward,
                              _backward_fn or _C.chamfer_distance_backward_cuda)
