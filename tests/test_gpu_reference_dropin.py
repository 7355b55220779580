"""Drop-in proof on the reference's own Python: the UNMODIFIED ``torkit3d/ops/*.py`` of a reference
install run on top of ``torkit3d_b200._C`` (the name ``torkit3d._C`` is made to resolve to the ctypes
shim before the operators are imported), and the reference's own ``tests/ops/test_*.py`` are executed
against that stack, parameter set by parameter set, with no edit to any reference file.

The reference install is looked up in ``$TK3D_REFERENCE`` (a checkout: ``torkit3d/`` and ``tests/ops/``
side by side), else in the git-ignored ``baseline/_ref/`` that ``__graft_entry__.build()`` fills
(``pip install --target`` of the reference plus a copy of its ``tests/`` folder).  Without either the
module is skipped.

Reference test files run here: ``tests/ops/test_knn_distance.py`` (float64, ``sorted=True``, incl. the
(32, 2048, 8192, k=64) case), ``test_sample_farthest_points.py``, ``test_ball_query.py``,
``test_chamfer_distance.py`` (incl. its ``gradcheck``), ``test_group_points.py``,
``test_interpolate_feature.py``.
"""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

REF_TEST_FILES = (
    "test_knn_distance.py",
    "test_sample_farthest_points.py",
    "test_ball_query.py",
    "test_chamfer_distance.py",
    "test_group_points.py",
    "test_interpolate_feature.py",
)


def _find_reference():
    cands = []
    if os.environ.get("TK3D_REFERENCE"):
        cands.append(os.environ["TK3D_REFERENCE"])
    cands.append(os.path.join(ROOT, "baseline", "_ref"))
    for c in cands:
        if (os.path.isfile(os.path.join(c, "torkit3d", "ops", "knn_points.py"))
                and os.path.isdir(os.path.join(c, "tests", "ops"))):
            return c
    return None


REF = _find_reference()
if REF is None:
    pytest.skip("no reference install (set TK3D_REFERENCE or run __graft_entry__.build() beside a checkout)",
                allow_module_level=True)


def _install_shim():
    """``torkit3d`` = the reference's pure-Python package, ``torkit3d._C`` = this repository's shim."""
    import torkit3d_b200._C as shim

    stale = [m for m in sys.modules if m == "torkit3d" or m.startswith("torkit3d.")]
    for m in stale:
        mod = sys.modules[m]
        if not getattr(mod, "__file__", "") or not str(mod.__file__).startswith(REF):
            del sys.modules[m]
    sys.modules["torkit3d._C"] = shim
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import torkit3d

    assert os.path.dirname(os.path.abspath(torkit3d.__file__)) == os.path.join(os.path.abspath(REF), "torkit3d")
    torkit3d._C = shim
    return shim


def _load_ref_tests():
    shim = _install_shim()
    cases = []
    for fname in REF_TEST_FILES:
        path = os.path.join(REF, "tests", "ops", fname)
        spec = importlib.util.spec_from_file_location("tk3d_reference_tests_" + fname[:-3], path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        for name in sorted(vars(mod)):
            fn = getattr(mod, name)
            if not name.startswith("test") or not callable(fn):
                continue
            param = [m for m in getattr(fn, "pytestmark", []) if m.name == "parametrize"]
            if not param:
                cases.append(pytest.param(fn, (), id="%s::%s" % (fname, name)))
                continue
            assert len(param) == 1
            for values in param[0].args[1]:
                cases.append(pytest.param(fn, tuple(values),
                                          id="%s::%s[%s]" % (fname, name, "-".join(str(v) for v in values))))
    return shim, cases


SHIM, CASES = _load_ref_tests()


def test_reference_ops_are_bound_to_the_shim():
    """Every reference operator module sees the ctypes shim as its ``_C`` (no file of the reference changed)."""
    import torkit3d.ops.ball_query as bq
    import torkit3d.ops.chamfer_distance as cd
    import torkit3d.ops.group_points as gp
    import torkit3d.ops.interpolate_feature as itp
    import torkit3d.ops.knn_points as kp
    import torkit3d.ops.sample_farthest_points as sfp

    for mod in (bq, cd, gp, itp, kp, sfp):
        assert mod._C is SHIM
        assert os.path.abspath(mod.__file__).startswith(os.path.abspath(REF))
    assert len(CASES) >= 25


@pytest.mark.gpu
@pytest.mark.parametrize("fn,args", CASES)
def test_reference_own_test(fn, args):
    import torch

    torch.manual_seed(0)
    fn(*args)
    torch.cuda.synchronize()
