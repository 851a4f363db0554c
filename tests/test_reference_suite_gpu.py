"""Runs the reference project's own test file (tests/test_causal_conv1d.py, all of it,
unmodified) against this package's CUDA kernels.

The file itself is not part of this repository: ``tests/reference_suite/prepare.py`` stages
a copy under ``baseline/_ref/reference_tests/`` together with a conftest that registers this
package under the reference's module names.  Without the staged copy the test is skipped.
The copy runs in a child pytest process (its conftest rewires ``sys.modules``).
"""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join(ROOT, "baseline", "_ref", "reference_tests")


@pytest.mark.gpu
def test_reference_projects_own_suite_passes():
    if not os.path.isfile(os.path.join(STAGED, "test_causal_conv1d.py")):
        pytest.skip("reference test file not staged (python tests/reference_suite/prepare.py <reference checkout>)")
    env = dict(os.environ, CC1D_REPO_ROOT=ROOT)
    res = subprocess.run([sys.executable, "-m", "pytest", STAGED, "-q", "--maxfail", "50", "-p", "no:cacheprovider",
                          "--rootdir", STAGED, "-c", os.devnull],
                         cwd=STAGED, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    tail = "\n".join(res.stdout.splitlines()[-25:])
    log_dir = os.environ.get("CC1D_TEST_LOG_DIR")       # optional: keep the child's full output
    if log_dir and os.path.isdir(log_dir):
        with open(os.path.join(log_dir, "reference_suite.log"), "w") as f:
            f.write(res.stdout)
    assert res.returncode == 0, f"the reference's own tests failed against this package:\n{tail}"
    m = re.search(r"(\d+) passed", res.stdout)
    assert m and int(m.group(1)) > 5000, f"unexpectedly few tests ran:\n{tail}"
    print(tail)
