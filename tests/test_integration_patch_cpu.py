"""The backend registration that ships as ``integration/trimul_b200_backend.patch`` applies to the
reference tree and does what INTEGRATION.md says: ``ImplementationType("b200")`` exists, resolves to
``KernelBackend.B200`` for the triangle multiplication (and to the PyTorch reference for every other
op), keeps fp32 inputs on the backend, builds ``TriangleMultiplication(implementation="b200")``, and
leaves the reference's own dispatch tests green.

Needs the reference checkout (``MINIWORLD_REFERENCE`` or ``reference_path`` in BASELINE.json);
skipped where it is absent.  Works on a temporary copy: the reference tree is never written to.
"""

import json
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATCH = os.path.join(ROOT, "integration", "trimul_b200_backend.patch")


def _reference_root():
    cand = os.environ.get("MINIWORLD_REFERENCE")
    if not cand:
        try:
            with open(os.path.join(ROOT, "BASELINE.json")) as f:
                cand = json.load(f).get("reference_path")
        except OSError:
            cand = None
    if cand and os.path.isdir(os.path.join(cand, "src", "miniworld_engine")):
        return cand
    return None


@pytest.fixture(scope="module")
def patched_tree(tmp_path_factory):
    ref = _reference_root()
    if ref is None:
        pytest.skip("reference checkout not available")
    if shutil.which("patch") is None:
        pytest.skip("patch(1) not installed")
    dst = tmp_path_factory.mktemp("patched_reference")
    shutil.copytree(os.path.join(ref, "src"), dst / "src", ignore=shutil.ignore_patterns("__pycache__"))
    os.makedirs(dst / "tests")
    shutil.copy(os.path.join(ref, "tests", "test_dispatch.py"), dst / "tests" / "test_dispatch.py")
    res = subprocess.run(["patch", "-p1", "--batch", "-i", PATCH], cwd=dst, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    return dst


def _run(tree, code):
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(tree / "src"), ROOT]))
    return subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=tree)


def test_backend_is_registered_and_resolves(patched_tree):
    code = r"""
import warnings, torch
from miniworld_engine.modules import dispatch
from miniworld_engine.modules.dispatch import KernelBackend
from miniworld_engine.modules.exceptions import ImplementationType
from miniworld_engine.modules.triangle_multiplication.module import TriangleMultiplication
assert ImplementationType("b200") is ImplementationType.B200
assert dispatch.to_kernel_backend(ImplementationType.B200) is KernelBackend.B200
assert dispatch.resolve_triangle_multiplication("b200") is KernelBackend.B200
assert dispatch.resolve_transition("b200") is KernelBackend.PYTORCH          # no such kernel: reference
with warnings.catch_warnings():
    warnings.simplefilter("error")                                            # fp32 and bf16 stay, no warning
    assert dispatch.guard_dtype(KernelBackend.B200, torch.float32, op="t") is KernelBackend.B200
    assert dispatch.guard_dtype(KernelBackend.B200, torch.bfloat16, op="t") is KernelBackend.B200
with warnings.catch_warnings():
    warnings.simplefilter("ignore")
    assert dispatch.guard_dtype(KernelBackend.B200, torch.float16, op="t") is KernelBackend.PYTORCH
m = TriangleMultiplication(32, implementation="b200")
assert m._backend is KernelBackend.B200 and hasattr(m, "_forward_b200")
# the branch reaches this package: on a CPU tensor the B200 path refuses (it has no CPU fallback)
try:
    with torch.no_grad():
        m(torch.zeros(1, 4, 4, 32))
except RuntimeError as e:
    assert "no CPU path" in str(e), e
else:
    raise AssertionError("the b200 branch was not taken")
print("OK")
"""
    res = _run(patched_tree, code)
    assert res.returncode == 0 and "OK" in res.stdout, res.stdout + res.stderr


def test_reference_dispatch_tests_pass_on_the_patched_tree(patched_tree):
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(patched_tree / "src"), ROOT]))
    res = subprocess.run([sys.executable, "-m", "pytest", "tests/test_dispatch.py", "-q", "-x", "-p", "no:cacheprovider"],
                         env=env, capture_output=True, text=True, cwd=patched_tree)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
