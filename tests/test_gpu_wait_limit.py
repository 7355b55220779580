"""The one kernel that waits for other thread blocks (cluster FPS) gives up after a limit instead of
hanging: a diagnostic launch in which one warp per cluster sends nothing makes every wait of that
step run out; the rows are marked from that step on, the counter of expired waits moves, and the
next regular call computes the regular result (the context is intact)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("n,clouds", [(6000, 2), (40000, 1)])
def test_fps_cluster_wait_runs_out_and_context_survives(oracle, n, clouds):
    from torkit3d_b200 import _lib
    from torkit3d_b200.ops import sample_farthest_points

    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(n)
    p = rng.random((clouds, n, 3)).astype(np.float32)
    pts = torch.from_numpy(p).to(DEV)
    s, drop = 24, 7
    want = oracle.fps(p, s)

    # every warp sends: the diagnostic entry is a regular run
    idx = torch.full((clouds, s), -7, dtype=torch.int64, device=DEV)
    before = lib.tk3d_fps_expired_waits()
    assert before >= 0
    assert lib.tk3d_diag_fps_wait_limit(pts.data_ptr(), clouds, n, s, idx.data_ptr(), 50, -1, st) == 0
    torch.cuda.synchronize()
    np.testing.assert_array_equal(idx.cpu().numpy(), want)
    assert lib.tk3d_fps_expired_waits() == before

    # one warp per cluster is silent in step `drop`: every wait of that step runs into the 50 ms limit
    idx.fill_(-7)
    assert lib.tk3d_diag_fps_wait_limit(pts.data_ptr(), clouds, n, s, idx.data_ptr(), 50, drop, st) == 0
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    got = idx.cpu().numpy()
    np.testing.assert_array_equal(got[:, :drop], want[:, :drop])
    assert (got[:, drop:] == -1).all()
    assert lib.tk3d_fps_expired_waits() > before

    # the context is intact and the next regular call is right
    np.testing.assert_array_equal(sample_farthest_points(pts, s).cpu().numpy(), want)


def test_wait_limit_arguments_are_checked():
    from torkit3d_b200 import _lib

    lib = _lib.load()
    x = torch.zeros(1, 5000, 3, device=DEV)
    i = torch.zeros(1, 4, dtype=torch.int64, device=DEV)
    assert lib.tk3d_diag_fps_wait_limit(x.data_ptr(), 1, 5000, 4, i.data_ptr(), 0, -1, None) != 0      # limit too short
    assert lib.tk3d_diag_fps_wait_limit(x.data_ptr(), 1, 5000, 4, i.data_ptr(), 5000, -1, None) != 0   # too long
    assert lib.tk3d_diag_fps_wait_limit(x.data_ptr(), 1, 1000, 4, i.data_ptr(), 50, -1, None) != 0     # not a cluster size
    assert lib.tk3d_diag_fps_wait_limit(None, 1, 5000, 4, i.data_ptr(), 50, -1, None) != 0
