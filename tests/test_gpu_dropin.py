"""The drop-in check: the reference's own fabric tests, unchanged, run against this library.

tests/dropin/prepare.py lays a copy of the reference's pure-Python package and of its test files
out under baseline/_ref/ (git-ignored) and puts monoserve_b200.compat._C where the reference keeps
its compiled extension.  Here each copied test file runs in a process of its own with that folder
first on the path; every test must pass, the ones that drive the reference's K-split tiles (kinds 45 / 46)
included: this library runs such a tile as one symmetric K-range record per row block.
Skipped when the layout is absent (a checkout of the reference is needed to make it).
"""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

def run_reference_tests(name, select=None):
    path = os.path.join(REF, "tests", name)
    if not os.path.exists(path) or not os.path.exists(os.path.join(REF, "monoserve", "_C.py")):
        pytest.skip("no drop-in layout under baseline/_ref (tests/dropin/prepare.py makes it)")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([REF, ROOT, os.environ.get("PYTHONPATH", "")]))
    cmd = [sys.executable, "-m", "pytest", os.path.join("tests", name), "-v", "-p", "no:cacheprovider",
           "--timeout", "120", "--timeout-method", "thread"]
    if select:
        cmd += ["-k", select]
    r = subprocess.run(cmd, cwd=REF, env=env, capture_output=True, text=True, timeout=900)
    outcome = {}
    for m in re.finditer(r"::(\S+) (PASSED|FAILED|ERROR|SKIPPED)", r.stdout):
        outcome[m.group(1)] = m.group(2)
    assert outcome, r.stdout[-2000:] + r.stderr[-2000:]
    return outcome, r.stdout


def test_reference_mechanism_tests_pass_unchanged():
    """tests/test_fabric_core.py of the reference: DAG order and exactly-once, floors and borrowing,
    link slots bound the tiles in flight, epoch spread, iterations, program switch, dynamic region."""
    outcome, log = run_reference_tests("test_fabric_core.py")
    assert len(outcome) >= 8
    assert all(v == "PASSED" for v in outcome.values()), (outcome, log[-3000:])


def test_reference_gemm_tests_pass_unchanged():
    """tests/test_fabric_gemm.py of the reference: every case that uses the symmetric GEMM tile
    (bf16 and e4m3, HBM and pinned host operands, all epilogues, K ranges) and every case built on the
    K-split tiles of kinds 45 / 46 and their reduce passes unchanged."""
    outcome, log = run_reference_tests("test_fabric_gemm.py")
    assert len(outcome) >= 28
    wrong = {k: v for k, v in outcome.items() if v != "PASSED"}
    assert not wrong, (wrong, log[-3000:])


def test_reference_lifetime_test_passes_unchanged():
    """tests/test_fabric_lifetime.py::test_freeing_a_stopped_fabric_while_another_runs: freeing a
    stopped fabric never waits for another fabric's kernel (the deferred releases)."""
    outcome, log = run_reference_tests("test_fabric_lifetime.py", select="freeing")
    assert outcome == {"test_freeing_a_stopped_fabric_while_another_runs": "PASSED"}, (outcome, log[-3000:])
