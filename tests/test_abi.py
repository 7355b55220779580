"""CPU-only checks of the C ABI: the library loads, exports every symbol the header declares, and
rejects bad arguments with the documented status codes before touching the GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from torkit3d_b200 import _lib, build

    build.build()
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "tk3d.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tk3d_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from torkit3d_b200 import _lib

    names = _declared()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), n
        assert n in _lib.SIGNATURES, "ctypes prototype missing for " + n
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_strerror(lib):
    assert lib.tk3d_version() >= 100
    assert lib.tk3d_strerror(0) == b"ok"
    for code in range(1, 8):
        assert lib.tk3d_strerror(code) not in (b"ok", b"unknown error code")
    assert lib.tk3d_strerror(99) == b"unknown error code"


def test_argument_errors_need_no_gpu(lib):
    from torkit3d_b200._lib import F32

    fake = ctypes.c_void_p(256)  # never dereferenced: every call below fails validation first
    assert lib.tk3d_knn(fake, fake, 1, 8, 4, 5, fake, fake, F32, None) == 3      # k > N2
    assert b"exceeds" in lib.tk3d_last_error()
    assert lib.tk3d_knn(fake, fake, 1, 8, 4, 0, fake, fake, F32, None) == 3      # k < 1
    assert lib.tk3d_knn(fake, fake, 1, 8, 4, 2, fake, fake, 7, None) == 4        # dtype
    assert lib.tk3d_knn(None, fake, 1, 8, 4, 2, fake, fake, F32, None) == 1      # NULL
    assert lib.tk3d_knn(fake, fake, -1, 8, 4, 2, fake, fake, F32, None) == 2     # negative size
    assert lib.tk3d_fps(fake, 1, 8, 0, fake, None, 0, F32, None) == 3            # num_samples <= 0
    assert lib.tk3d_fps(fake, 1, 8, 9, fake, None, 0, F32, None) == 3            # num_samples > N
    assert lib.tk3d_fps(fake, 1, 100000, 9, fake, None, 0, F32, None) == 6       # scratch required
    assert lib.tk3d_fps_scratch_bytes(4, 16384, F32) == 0
    assert lib.tk3d_fps_scratch_bytes(4, 16385, F32) == 4 * 16385 * 4
    assert lib.tk3d_fps_scratch_bytes(4, 8192, 1) == 0            # fp64 clouds up to 8192 points are resident too
    assert lib.tk3d_fps_scratch_bytes(4, 8193, 1) == 4 * 8193 * 8
    assert lib.tk3d_ball_query(fake, fake, 1, 8, 8, 0.1, 0, fake, F32, None) == 3
    assert lib.tk3d_interp_fwd(fake, fake, fake, 1, 1, 8, 8, 4, fake, None, None, 0, F32, None) == 3  # k != 3
    assert lib.tk3d_chamfer_fwd(None, fake, 1, 8, 8, fake, fake, fake, fake, None, F32, None) == 1
    assert lib.tk3d_three_nn_weight(fake, 4, 9, fake, F32, None) == 3
    assert lib.tk3d_feature_knn(fake, fake, 1, 16, 8, 4, 5, 1, fake, fake, F32, None) == 3     # k > N2
    assert lib.tk3d_feature_knn(fake, fake, 1, 16, 8, 400, 129, 1, fake, fake, F32, None) == 7  # k > 128
    assert lib.tk3d_feature_knn(fake, fake, 1, 16, 8, 4, 2, 1, fake, fake, 1, None) == 7        # float64
    assert lib.tk3d_feature_knn(fake, fake, 1, 0, 8, 4, 2, 1, fake, fake, F32, None) == 2       # no channels
    assert lib.tk3d_feature_knn(fake, None, 1, 16, 8, 4, 2, 1, fake, fake, F32, None) == 1      # NULL
    assert lib.tk3d_feature_knn(None, None, 0, 16, 8, 4, 2, 1, None, None, F32, None) == 0      # empty batch
    # which forward kernel a chamfer call would launch (one string per regime; fp64 has one kernel)
    names = {lib.tk3d_chamfer_fwd_kernel_name(b, 16384, 16384, F32) for b in (1, 2, 8, 16, 24, 64)}
    assert names <= {b"chamfer_fwd_fast_kernel<1>", b"chamfer_fwd_smwide_kernel", b"chamfer_fwd_fast_kernel<2>"}
    assert lib.tk3d_chamfer_fwd_kernel_name(2, 1024, 1024, F32) == b"chamfer_fwd_fast_kernel<1>"
    assert lib.tk3d_chamfer_fwd_kernel_name(2, 1024, 1024, 1) == b"chamfer_fwd_generic_kernel"
    # empty problems succeed without launching anything
    assert lib.tk3d_knn(None, None, 0, 8, 4, 2, None, None, F32, None) == 0
    assert lib.tk3d_group_fwd(None, None, 0, 4, 8, 8, 2, None, None, None, 0, F32, None) == 0
    # the row-gather path wants scratch only when the output dwarfs the features; shapes the channel-row
    # kernel serves (N1 a multiple of 4 up to 24576, at least 1024 entries per cloud) need none
    assert lib.tk3d_group_fwd_scratch_bytes(32, 64, 8192, 1024, 32, F32) == 0
    assert lib.tk3d_group_fwd_scratch_bytes(32, 64, 32768, 4096, 32, F32) == 32 * 64 * 32768 * 4
    assert lib.tk3d_group_bwd_scratch_bytes(32, 64, 8192, 1024, 32, F32) == 32 * 64 * 8192 * 4
    assert lib.tk3d_group_fwd_scratch_bytes(32, 64, 8192, 16, 4, F32) == 0
    assert lib.tk3d_group_fwd_scratch_bytes(32, 64, 8192, 1024, 32, 1) == 0
    assert lib.tk3d_interp_fwd_scratch_bytes(8, 128, 32768, 131072, F32) == 8 * 128 * 32768 * 4
    assert lib.tk3d_interp_fwd_scratch_bytes(8, 4, 32768, 131072, F32) == 0


def test_shim_rejects_cpu_tensors():
    import torch

    from torkit3d_b200 import _C

    x = torch.zeros(1, 8, 3)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        _C.knn_distance_cuda(x, x, 2, 1)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        _C.sample_farthest_points_cuda(x, 2)
    with pytest.raises(AssertionError, match="Only support cuda"):
        from torkit3d_b200.ops import chamfer_distance

        chamfer_distance(x, x)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from torkit3d_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.load()
