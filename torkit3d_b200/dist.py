"""Multi-GPU use of the operators: one process per GPU, independent shards, one scalar exchange.

Every operator of this package is independent per cloud (batch entry) and -- except farthest point
sampling -- per query point, so a job scales by giving each rank a slice of the batch
(``batch_shard``) or, for a single huge scene, a slab of the query points (``query_slab``) with the
key cloud and its features replicated.  No operator needs another rank's data.  The only exchange
is the scalar chamfer loss: ``chamfer_loss`` (autograd) and ``chamfer_step`` (loss and gradients
in one call, gradient kernels overlapped with the collective) produce the local partial sums
inside the forward kernel's epilogue and all-reduce two float64 numbers (NCCL over NVLink when the tensors are on
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
        fused = forward_fn is None and backward_fn is None  # the library's own loss/gradient entry points
        # the library's forward clears the sums itself; the stand-ins of the host-logic tests accumulate
        sums = (torch.empty if fused else torch.zeros)(2, dtype=torch.float64, device=a.device)
        _, idx1, _, idx2 = (forward_fn or _cuda_forward)(a, b, sums)
        if _world(group) > 1:
            dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
        ctx.save_for_backward(a, b, idx1, idx2)
        ctx.counts = (count1, count2)
        ctx.backward_fn = backward_fn
        if fused:
            from . import _lib
            from ._C import _dtype, _on, _ptr, _stream

            loss = torch.empty((), dtype=a.dtype, device=a.device)
            with _on(a.device):
                _lib.check(_lib.load().tk3d_chamfer_mean_loss(_ptr(sums), count1, count2, _ptr(loss), _dtype(a),
                                                              _stream(a)))
            return loss
        loss = sums[0] / count1 + sums[1] / count2
        return loss.to(a.dtype)

    @staticmethod
    def backward(ctx, grad_loss):
        a, b, idx1, idx2 = ctx.saved_tensors
        c1, c2 = ctx.counts
        if ctx.backward_fn is None:
            # one launch pair: the constant upstream gradients grad_loss/count are formed inside the kernels
            from . import _lib
            from ._C import _dtype, _on, _ptr, _stream

            gl = grad_loss.to(a.dtype).contiguous()
            ga, gb = torch.empty_like(a), torch.empty_like(b)
            with _on(a.device):
                _lib.check(_lib.load().tk3d_chamfer_bwd_mean(_ptr(gl), c1, c2, _ptr(a), _ptr(b), _ptr(idx1), _ptr(idx2),
                                                             a.size(0), a.size(1), b.size(1), _ptr(ga), _ptr(gb),
                                                             _dtype(a), _stream(a)))
            return ga, gb, None, None, None, None, None
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
    if (_forward_fn is None) != (_backward_fn is None):  # host-logic tests replace both or neither
        _forward_fn = _forward_fn or _cuda_forward
        _backward_fn = _backward_fn or _C.chamfer_distance_backward_cuda
    return _ChamferLoss.apply(xyz1, xyz2, count1, count2, group, _forward_fn, _backward_fn)


_ones = {}


def _one(device, dtype):
    """A cached device scalar 1 (the upstream gradient of a loss); filled once, never written again."""
    key = (device.type, device.index, dtype)
    t = _ones.get(key)
    if t is None:
        t = torch.ones((), dtype=dtype, device=device)
        _ones[key] = t
    return t


# ---- training step without autograd ---------------------------------------------------------------
def chamfer_step(xyz1, xyz2, global_batch=None, group=None, workspace=None):
    """Mean chamfer loss over a batch sharded across ranks AND its gradients, in one call.

    The loss is linear in the per-point distances, so the gradient kernels need only the counts,
    not the reduced loss: they are launched right behind the forward kernel while the all-reduce of
    the two partial sums is in flight (``async_op``), and only the final loss kernel waits for it.
    Five launches per step (forward, two gradient kernels, the collective, the loss), no
    element-wise PyTorch kernel, no autograd graph.

    Args:
        xyz1: [B_local, N1, 3] float32/float64 CUDA tensor, this rank's clouds;  xyz2: [B_local, N2, 3].
        global_batch, group: as for ``chamfer_loss``.
        workspace: optional dict owned by the caller.  The outputs and intermediate tensors of the
            step are then kept in it and reused by the next call with the same shapes (ten fewer
            allocations per step, which matters when a step takes less than a millisecond); the
            tensors returned by one call are overwritten by the next call with that workspace.

    Returns:
        (loss, grad_xyz1, grad_xyz2): the global mean loss (0-dim, identical on every rank) and
        its gradients w.r.t. this rank's clouds.
    """
    from . import _lib
    from ._C import _dtype, _on, _ptr, _stream

    a, b = xyz1.detach().contiguous(), xyz2.detach().contiguous()
    lib = _lib.load()
    world = _world(group)
    B, n1, n2 = a.size(0), a.size(1), b.size(1)
    gbatch = int(global_batch) if global_batch is not None else B * world
    count1, count2 = float(gbatch * n1), float(gbatch * n2)
    dev, dt = a.device, _dtype(a)
    with _on(dev):
        st = _stream(a)
        key = (B, n1, n2, a.dtype, dev)
        bufs = workspace.get(key) if workspace is not None else None
        if bufs is None:
            bufs = (torch.empty((B, n1), dtype=a.dtype, device=dev), torch.empty((B, n2), dtype=a.dtype, device=dev),
                    torch.empty((B, n1), dtype=torch.int64, device=dev),
                    torch.empty((B, n2), dtype=torch.int64, device=dev), torch.empty_like(a), torch.empty_like(b),
                    torch.empty(2, dtype=torch.float64, device=dev), torch.empty((), dtype=a.dtype, device=dev))
            if workspace is not None:
                workspace[key] = bufs
        d1, d2, i1, i2, ga, gb, sums, loss = bufs
        one = _one(dev, a.dtype)
        _lib.check(lib.tk3d_chamfer_fwd(_ptr(a), _ptr(b), B, n1, n2, _ptr(d1), _ptr(i1), _ptr(d2), _ptr(i2),
                                        _ptr(sums), dt, st))
        work = dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group, async_op=True) if world > 1 else None
        _lib.check(lib.tk3d_chamfer_bwd_mean(_ptr(one), count1, count2, _ptr(a), _ptr(b), _ptr(i1), _ptr(i2), B, n1,
                                             n2, _ptr(ga), _ptr(gb), dt, st))
        if work is not None:
            work.wait()  # the current stream waits for the collective; the host does not
        _lib.check(lib.tk3d_chamfer_mean_loss(_ptr(sums), count1, count2, _ptr(loss), dt, st))
    return loss, ga, gb


# ---- training step on host-resident clouds ------------------------------------------------------
_copy_streams = {}


def _copy_stream(device):
    """One side stream per device for host-to-device copies (created on first use)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _copy_streams:
        _copy_streams[key] = torch.cuda.Stream(device=device)
    return _copy_streams[key]


def chamfer_step_from_host(xyz1_host, xyz2_host, device, global_batch=None, group=None, chunks=1):
    """Chamfer loss and its gradients for clouds that live in (pinned) host memory.

    With ``chunks`` > 1 the batch is cut into slices; slice i+1 is copied to the GPU on a side
    stream while the forward and backward kernels of slice i run on the current stream.  This is
    possible because the mean loss is linear in the per-point distances: d loss / d dist is the
    constant 1/count, known before any distance is, so each slice's gradient kernels can run right
    after its forward kernel.  Slicing adds launches and host work per slice: on B200, 64 pairs of
    16384-point clouds in 8 slices ran slower (7.3 ms) than unsliced (6.85 ms).  To hide the copy of
    such batches use ``HostCloudPrefetcher`` across steps.

    Args:
        xyz1_host: [B_local, N1, 3] float32 CPU tensor (pin it for asynchronous copies).
        xyz2_host: [B_local, N2, 3].
        device: CUDA device of this rank.
        global_batch, group: as for ``chamfer_loss``.

    Returns:
        (loss, grad_xyz1, grad_xyz2): loss is a 0-dim float32 tensor on ``device`` (identical on
        every rank), the gradients are those of the global mean loss w.r.t. this rank's clouds.
    """
    from . import _lib
    from ._lib import check, load

    if xyz1_host.dtype != torch.float32 or xyz2_host.dtype != torch.float32:
        raise RuntimeError("chamfer_step_from_host: float32 clouds expected")
    if xyz1_host.dim() != 3 or xyz2_host.dim() != 3 or xyz1_host.size(2) != 3 or xyz2_host.size(2) != 3:
        raise RuntimeError("chamfer_step_from_host: clouds must be [B, N, 3]")
    if xyz1_host.size(0) != xyz2_host.size(0):
        raise RuntimeError("chamfer_step_from_host: batch sizes differ")
    xyz1_host, xyz2_host = xyz1_host.contiguous(), xyz2_host.contiguous()
    lib = load()
    dev = torch.device(device)
    B, n1, n2 = xyz1_host.size(0), xyz1_host.size(1), xyz2_host.size(1)
    world = _world(group)
    gb = int(global_batch) if global_batch is not None else B * world
    count1, count2 = float(gb * n1), float(gb * n2)
    nch = max(1, min(int(chunks), B)) if B > 0 else 1
    with torch.cuda.device(dev):
        compute = torch.cuda.current_stream(dev)
        copy = _copy_stream(dev)
        a = torch.empty((B, n1, 3), dtype=torch.float32, device=dev)
        b = torch.empty((B, n2, 3), dtype=torch.float32, device=dev)
        d1 = torch.empty((B, n1), dtype=torch.float32, device=dev)
        d2 = torch.empty((B, n2), dtype=torch.float32, device=dev)
        i1 = torch.empty((B, n1), dtype=torch.int64, device=dev)
        i2 = torch.empty((B, n2), dtype=torch.int64, device=dev)
        ga, gbt = torch.empty_like(a), torch.empty_like(b)
        sums = torch.zeros((nch, 2), dtype=torch.float64, device=dev)  # the kernel overwrites its row
        per = (B + nch - 1) // nch if B > 0 else 0
        one = _one(dev, torch.float32)  # upstream gradient of the loss
        copy.wait_stream(compute)  # the buffers above exist before the side stream writes them
        for t in (a, b):
            t.record_stream(copy)
        for c in range(nch):
            b0, b1 = c * per, min(B, (c + 1) * per)
            if b1 <= b0:
                break
            with torch.cuda.stream(copy):
                a[b0:b1].copy_(xyz1_host[b0:b1], non_blocking=True)
                b[b0:b1].copy_(xyz2_host[b0:b1], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(copy)
            compute.wait_event(ready)
            st = compute.cuda_stream
            check(lib.tk3d_chamfer_fwd(a[b0:b1].data_ptr(), b[b0:b1].data_ptr(), b1 - b0, n1, n2,
                                       d1[b0:b1].data_ptr(), i1[b0:b1].data_ptr(), d2[b0:b1].data_ptr(),
                                       i2[b0:b1].data_ptr(), sums[c].data_ptr(), _lib.F32, st))
            check(lib.tk3d_chamfer_bwd_mean(one.data_ptr(), count1, count2, a[b0:b1].data_ptr(),
                                            b[b0:b1].data_ptr(), i1[b0:b1].data_ptr(), i2[b0:b1].data_ptr(),
                                            b1 - b0, n1, n2, ga[b0:b1].data_ptr(), gbt[b0:b1].data_ptr(), _lib.F32,
                                            st))
        sums = sums[0] if nch == 1 else sums.sum(dim=0)
        if world > 1:
            dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        check(lib.tk3d_chamfer_mean_loss(sums.data_ptr(), count1, count2, loss.data_ptr(), _lib.F32,
                                         compute.cuda_stream))
    return loss, ga, gbt


class HostCloudPrefetcher:
    """Double-buffered staging of host-resident cloud pairs: the copy of the next batch runs on a
    side stream while the kernels of the current batch run on the compute stream.

    ``prefetch(h1, h2)`` enqueues the copies of one batch (pinned float32 CPU tensors [B,N,3]) into
    the free buffer pair; ``get()`` returns the device tensors of the oldest prefetched batch after
    making the current stream wait for its copy.  At most two batches are in flight; a buffer pair
    is reused only after the work that was on the compute stream when the FOLLOWING batch was
    fetched (the kernels that read the pair) has finished, so ``prefetch`` may be called before or
    after the current step's kernels are launched and its copy overlaps them either way.
    """

    def __init__(self, device):
        self.device = torch.device(device)
        self._slots = [None, None]
        self._events = [None, None]
        self._release = [None, None]  # per buffer pair: recorded when the other pair was fetched
        self._queue = []
        self._next = 0

    def prefetch(self, h1, h2):
        if len(self._queue) >= 2:
            raise RuntimeError("HostCloudPrefetcher: two batches are already in flight; call get() first")
        slot = self._next
        self._next ^= 1
        with torch.cuda.device(self.device):
            compute = torch.cuda.current_stream(self.device)
            copy = _copy_stream(self.device)
            bufs = self._slots[slot]
            if bufs is None or bufs[0].shape != h1.shape or bufs[1].shape != h2.shape:
                bufs = (torch.empty(h1.shape, dtype=h1.dtype, device=self.device),
                        torch.empty(h2.shape, dtype=h2.dtype, device=self.device))
                for t in bufs:
                    t.record_stream(copy)
                self._slots[slot] = bufs
                copy.wait_stream(compute)  # fresh memory may have belonged to work still queued there
            elif self._release[slot] is not None:
                copy.wait_event(self._release[slot])  # the readers of this buffer pair are done
            with torch.cuda.stream(copy):
                bufs[0].copy_(h1, non_blocking=True)
                bufs[1].copy_(h2, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy)
            self._events[slot] = ev
            self._queue.append(slot)

    def get(self):
        if not self._queue:
            raise RuntimeError("HostCloudPrefetcher: nothing was prefetched")
        slot = self._queue.pop(0)
        compute = torch.cuda.current_stream(self.device)
        # whatever read the other buffer pair has been enqueued by now
        released = torch.cuda.Event()
        released.record(compute)
        self._release[slot ^ 1] = released
        compute.wait_event(self._events[slot])
        return self._slots[slot]
