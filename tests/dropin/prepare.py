"""Lay out the drop-in check: a copy of the reference's pure-Python package `monoserve/` and of
its fabric test files under baseline/_ref/ (git-ignored), with this library standing where the
reference keeps its compiled extension: baseline/_ref/monoserve/_C.py re-exports
monoserve_b200.compat._C.  Nothing of the reference is changed; one file is added.

    MONOSERVE_REFERENCE=<checkout of the reference> python tests/dropin/prepare.py

tests/test_gpu_dropin.py then runs the copied test files, unchanged, against libmonofab.
"""
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
DEST = os.path.join(ROOT, "baseline", "_ref")
TESTS = ["test_fabric_core.py", "test_fabric_gemm.py", "test_fabric_lifetime.py"]
SHIM = '''"""Stands where the reference keeps its compiled extension (added by tests/dropin/prepare.py)."""
from monoserve_b200.compat._C import *  # noqa: F401,F403
from monoserve_b200.compat._C import control  # noqa: F401
'''


def main():
    ref = os.environ.get("MONOSERVE_REFERENCE")
    if not ref or not os.path.isdir(os.path.join(ref, "monoserve")):
        sys.exit("set MONOSERVE_REFERENCE to a checkout of the reference project")
    pkg = os.path.join(DEST, "monoserve")
    if os.path.isdir(pkg):
        shutil.rmtree(pkg)
    shutil.copytree(os.path.join(ref, "monoserve"), pkg, ignore=shutil.ignore_patterns("__pycache__", "*.so"))
    with open(os.path.join(pkg, "_C.py"), "w") as f:
        f.write(SHIM)
    os.makedirs(os.path.join(DEST, "tests"), exist_ok=True)
    for name in TESTS:
        shutil.copy(os.path.join(ref, "tests", name), os.path.join(DEST, "tests", name))
    print("drop-in check laid out under", DEST)


if __name__ == "__main__":
    main()
