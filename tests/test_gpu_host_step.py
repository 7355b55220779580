"""chamfer_step_from_host: copies overlapped with the kernels slice by slice must give the loss
and gradients of the one-shot autograd path (sums are accumulated in float64; the gradients'
float atomics reorder, hence rel 1e-5 / abs 1e-6 there)."""
import pytest
import torch

from torkit3d_b200 import workloads
from torkit3d_b200.dist import HostCloudPrefetcher, chamfer_loss, chamfer_step_from_host

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("B,chunks", [(8, 4), (7, 3), (2, 8), (1, 1)])
def test_host_step_matches_autograd(B, chunks):
    x1, x2 = workloads.c4_chamfer_large(B=B, N=1500, M=1300, seed=5)
    h1, h2 = x1.pin_memory(), x2.pin_memory()
    loss, g1, g2 = chamfer_step_from_host(h1, h2, DEV, chunks=chunks)
    a = x1.to(DEV).requires_grad_(True)
    b = x2.to(DEV).requires_grad_(True)
    ref = chamfer_loss(a, b)
    ref.backward()
    torch.testing.assert_close(loss, ref.detach(), rtol=1e-6, atol=0)
    torch.testing.assert_close(g1, a.grad, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(g2, b.grad, rtol=1e-5, atol=1e-6)


def test_host_step_global_batch_scaling():
    x1, x2 = workloads.c4_chamfer_large(B=4, N=512, M=640, seed=6)
    loss, g1, _ = chamfer_step_from_host(x1.pin_memory(), x2.pin_memory(), DEV, global_batch=8, chunks=2)
    loss1, h1, _ = chamfer_step_from_host(x1.pin_memory(), x2.pin_memory(), DEV, chunks=2)
    torch.testing.assert_close(loss * 2, loss1, rtol=1e-6, atol=0)
    torch.testing.assert_close(g1 * 2, h1, rtol=1e-5, atol=1e-9)  # float atomics reorder between runs


def test_host_step_rejects_bad_input():
    with pytest.raises(RuntimeError):
        chamfer_step_from_host(torch.zeros(2, 8, 3, dtype=torch.float64), torch.zeros(2, 8, 3, dtype=torch.float64), DEV)
    with pytest.raises(RuntimeError):
        chamfer_step_from_host(torch.zeros(2, 8, 3), torch.zeros(3, 8, 3), DEV)


def test_prefetcher_double_buffer():
    pf = HostCloudPrefetcher(DEV)
    batches = [workloads.c4_chamfer_large(B=3, N=700, M=600, seed=10 + i) for i in range(4)]
    pinned = [(a.pin_memory(), b.pin_memory()) for a, b in batches]
    pf.prefetch(*pinned[0])
    for i in range(4):
        a, b = pf.get()
        if i + 1 < 4:
            pf.prefetch(*pinned[i + 1])
        loss = chamfer_loss(a, b)
        ref = chamfer_loss(batches[i][0].to(DEV), batches[i][1].to(DEV))
        assert torch.equal(a.cpu(), batches[i][0]) and torch.equal(b.cpu(), batches[i][1])
        torch.testing.assert_close(loss, ref, rtol=1e-6, atol=0)
    with pytest.raises(RuntimeError):
        pf.get()


def test_prefetcher_prefetch_behind_the_step_and_workspace():
    """The next batch may be requested after the current step's kernels were launched (its copy must
    not overwrite what they still read), and a workspace makes chamfer_step reuse its tensors."""
    from torkit3d_b200.dist import chamfer_step

    pf = HostCloudPrefetcher(DEV)
    batches = [workloads.c4_chamfer_large(B=4, N=3000, M=2500, seed=30 + i) for i in range(6)]
    pinned = [(a.pin_memory(), b.pin_memory()) for a, b in batches]
    ws = {}
    losses, ptrs = [], set()
    pf.prefetch(*pinned[0])
    for i in range(6):
        a, b = pf.get()
        loss, ga, _ = chamfer_step(a, b, workspace=ws)
        if i + 1 < 6:
            pf.prefetch(*pinned[i + 1])
        losses.append(float(loss))          # reads the result before the next call overwrites it
        ptrs.add(ga.data_ptr())
    assert len(ptrs) == 1 and len(ws) == 1   # one set of tensors, reused
    for i in range(6):
        ref, _, _ = chamfer_step(batches[i][0].to(DEV), batches[i][1].to(DEV))
        assert abs(losses[i] - float(ref)) <= 1e-6 * abs(float(ref))


@pytest.mark.parametrize("dt", [torch.float32, torch.float64])
def test_chamfer_step_matches_autograd(dt):
    """dist.chamfer_step (loss + gradients in one call, no autograd graph) against chamfer_loss + backward."""
    from torkit3d_b200.dist import chamfer_step

    x1, x2 = workloads.c4_chamfer_large(B=5, N=1100, M=900, seed=8)
    a = x1.to(DEV, dt).requires_grad_(True)
    b = x2.to(DEV, dt).requires_grad_(True)
    ref = chamfer_loss(a, b, global_batch=10)
    ref.backward()
    loss, ga, gb = chamfer_step(a, b, global_batch=10)
    assert loss.dtype == dt and ga.shape == a.shape and gb.shape == b.shape
    tol = dict(rtol=1e-5, atol=1e-6) if dt == torch.float32 else dict(rtol=1e-10, atol=1e-12)
    torch.testing.assert_close(loss, ref.detach(), rtol=1e-6, atol=0)
    torch.testing.assert_close(ga, a.grad, **tol)
    torch.testing.assert_close(gb, b.grad, **tol)
    # a second call gives the same loss bit for bit (float64 sums, deterministic order inside a block aside,
    # the two sums are accumulated with float64 atomics: compare to 1e-12)
    loss2, _, _ = chamfer_step(a, b, global_batch=10)
    torch.testing.assert_close(loss2, loss, rtol=1e-6, atol=0)
