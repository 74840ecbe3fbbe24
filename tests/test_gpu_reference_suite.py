"""The reference project's OWN test files, unmodified, run against this package on the GPU.

``__graft_entry__.build()`` copies the reference's ``tests/`` directory into the git-ignored
``baseline/_ref/reference_tests/`` when the reference tree is present; the files travel with the
repository from there.  They import ``spline_kan``, which resolves to this repository's alias
package (the directory the tests sit in holds no package of that name), so every assertion in them
-- tolerances included -- is checked against the B200 kernels.  ``test_experimental.py`` is left out:
it covers the reference's opt-in experimental layers, which are not part of the accelerated path.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SUITE = os.path.join(ROOT, "baseline", "_ref", "reference_tests")
FILES = ["test_cuda.py", "test_local_basis.py", "test_fused_regularization.py", "test_math_correctness.py",
         "test_reference.py", "test_corrections.py", "test_pruning.py", "test_grid_extension.py", "test_export.py"]


@pytest.mark.parametrize("name", FILES)
def test_reference_test_file_passes_against_this_package(name):
    path = os.path.join(SUITE, "tests", name)
    if not os.path.exists(path):
        pytest.skip("the reference's test files are not present (baseline/_ref/reference_tests)")
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join("tests", name), "-q", "-x", "-p",
                        "no:cacheprovider", "-W", "ignore"], cwd=SUITE, env=env, capture_output=True, text=True,
                       timeout=1500)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    # the file must really have run on the GPU against this package: no wholesale skip
    summary = [ln for ln in r.stdout.splitlines() if " passed" in ln]
    assert summary, tail
    print(name, summary[-1])
