"""ctypes binding of libtk3d_b200.so (the C ABI declared in include/tk3d.h).

The library is the product: there is no fallback.  If it is missing, or a call is made without a
CUDA device, the operators raise instead of computing anything on the CPU.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libtk3d_b200.so")

F32, F64 = 0, 1
I64, I32 = 0, 1

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p
_int = ctypes.c_int

# name -> (restype, argtypes); mirrors include/tk3d.h one to one
SIGNATURES = {
    "tk3d_version": (_int, []),
    "tk3d_strerror": (ctypes.c_char_p, [_int]),
    "tk3d_last_error": (ctypes.c_char_p, []),
    "tk3d_chamfer_fwd": (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "tk3d_chamfer_bwd": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _int, _vp]),
    "tk3d_chamfer_mean_loss": (_int, [_vp, ctypes.c_double, ctypes.c_double, _vp, _int, _vp]),
    "tk3d_chamfer_bwd_mean": (_int, [_vp, ctypes.c_double, ctypes.c_double, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                     _vp, _vp, _int, _vp]),
    "tk3d_knn": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _int, _vp]),
    "tk3d_fps_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _int]),
    "tk3d_fps": (_int, [_vp, _i64, _i64, _i64, _vp, _vp, ctypes.c_size_t, _int, _vp]),
    "tk3d_fps_static_scratch_capacity": (ctypes.c_size_t, []),
    "tk3d_fps_static_scratch": (_int, [_vp, _i64, _i64, _i64, _vp, _int, _vp]),
    "tk3d_ball_query": (_int, [_vp, _vp, _i64, _i64, _i64, ctypes.c_float, _i64, _vp, _int, _vp]),
    "tk3d_group_fwd_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _i64, _i64, _int]),
    "tk3d_group_fwd": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, ctypes.c_size_t, _int, _vp]),
    "tk3d_group_bwd_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _i64, _i64, _int]),
    "tk3d_group_bwd": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, ctypes.c_size_t, _int, _vp]),
    "tk3d_interp_fwd_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _i64, _int]),
    "tk3d_interp_fwd": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, ctypes.c_size_t, _int,
                               _vp]),
    "tk3d_interp_bwd_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _i64, _int]),
    "tk3d_interp_bwd": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, ctypes.c_size_t, _int,
                               _vp]),
    "tk3d_three_nn_weight": (_int, [_vp, _i64, _i64, _vp, _int, _vp]),
    "tk3d_fps_gather": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, ctypes.c_size_t, _int, _vp]),
    "tk3d_sa_group_supported": (_int, [_i64, _i64, _i64, _i64, _i64, _int]),
    "tk3d_sa_group_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _i64, _i64, _int]),
    "tk3d_sa_group_fwd": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, ctypes.c_float, _i64, _int, _int, _vp, _vp,
                                 _vp, _vp, ctypes.c_size_t, _int, _vp]),
    "tk3d_sa_group_bwd": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp, _vp, _vp,
                                 ctypes.c_size_t, _int, _vp]),
    "tk3d_three_nn_interp_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _i64, _int]),
    "tk3d_three_nn_interp_fwd": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, ctypes.c_float, _vp, _vp, _vp,
                                        _vp, _vp, ctypes.c_size_t, _int, _vp]),
    "tk3d_three_nn_interp_bwd": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp, ctypes.c_size_t, _int,
                                        _vp]),
    "tk3d_edge_feature_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _i64, _i64, _int]),
    "tk3d_edge_feature_fwd": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp,
                                     ctypes.c_size_t, _int, _vp]),
    "tk3d_edge_feature_bwd": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp,
                                     ctypes.c_size_t, _int, _vp]),
    "tk3d_bounds_violations": (ctypes.c_longlong, []),
    "tk3d_fps_expired_waits": (ctypes.c_longlong, []),
    "tk3d_diag_fps_wait_limit": (_int, [_vp, _i64, _i64, _i64, _vp, _i64, _i64, _vp]),
    "tk3d_diag_ffma": (_int, [_i64, _vp, ctypes.POINTER(ctypes.c_double), _vp]),
    "tk3d_feature_knn": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _vp, _vp, _int, _vp]),
    "tk3d_chamfer_fwd_kernel_name": (ctypes.c_char_p, [_i64, _i64, _i64, _int]),
    # layout variants: [B,3,N] coordinates read in place, optional int32 index tensors
    "tk3d_chamfer_fwd_layout": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "tk3d_chamfer_bwd_layout": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _int, _vp]),
    "tk3d_chamfer_bwd_mean_layout": (_int, [_vp, ctypes.c_double, ctypes.c_double, _vp, _vp, _vp, _vp, _i64, _i64,
                                            _i64, _int, _vp, _vp, _int, _vp]),
    "tk3d_knn_layout": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp, _int, _int, _vp]),
    "tk3d_fps_layout": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, ctypes.c_size_t, _int, _vp]),
    "tk3d_ball_query_layout": (_int, [_vp, _vp, _i64, _i64, _i64, ctypes.c_float, _i64, _int, _vp, _int, _int, _vp]),
    "tk3d_feature_rows": (_int, [_vp, _i64, _i64, _i64, _vp, _int, _vp]),
    "tk3d_interp_fwd_rows": (_int, [_vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _int, _vp]),
    "tk3d_group_fwd_rows": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _int, _vp]),
    "tk3d_group_fwd_layout": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, ctypes.c_size_t, _int,
                                     _vp]),
}

_lib = None


def load():
    """Load the shared library (once) and attach the prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libtk3d_b200.so is not built (expected at %s). Run `python -m torkit3d_b200.build`; "
            "there is no CPU or PyTorch fallback." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def load_bounds_checked():
    """The range-checked build (libtk3d_b200_bounds.so, ``python -m torkit3d_b200.build --bounds``) with the
    same prototypes attached -- test infrastructure: the operators never load it."""
    path = os.path.join(_PKG, "libtk3d_b200_bounds.so")
    if not os.path.exists(path):
        raise ImportError("libtk3d_b200_bounds.so is not built (python -m torkit3d_b200.build --bounds)")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


def check(rc):
    """Turn a non-zero status into RuntimeError (what TORCH_CHECK raises in the reference)."""
    if rc != 0:
        lib = load()
        detail = lib.tk3d_last_error().decode()
        raise RuntimeError("tk3d: %s%s" % (lib.tk3d_strerror(rc).decode(), (": " + detail) if detail else ""))


_scratch_cache = {}


def scratch_bytes(name, *args):
    """Result of the library's ``<name>_scratch_bytes(*args)`` query, memoised per argument tuple
    (the answer depends on the shape only; repeated calls of one shape skip a foreign-function call)."""
    key = (name,) + args
    v = _scratch_cache.get(key)
    if v is None:
        if len(_scratch_cache) > 4096:
            _scratch_cache.clear()
        v = int(getattr(load(), name + "_scratch_bytes")(*args))
        _scratch_cache[key] = v
    return v
