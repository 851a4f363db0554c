#!/usr/bin/env python
"""Stage the reference project's own test file so that it can run against this package.

    python tests/reference_suite/prepare.py <path to a checkout of Dao-AILab/causal-conv1d>

Copies ``<checkout>/tests/test_causal_conv1d.py`` UNMODIFIED into
``baseline/_ref/reference_tests/`` (git-ignored: the reference's sources never enter this
repository's history) and puts ``reference_conftest.py`` beside it as ``conftest.py``.  Then

    python -m pytest baseline/_ref/reference_tests -q

runs the reference's whole parity suite against the CUDA kernels of this package;
``tests/test_reference_suite_gpu.py`` does exactly that when the staged copy is present.
"""
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
DEST = os.path.join(ROOT, "baseline", "_ref", "reference_tests")


def main(argv):
    if len(argv) != 2:
        raise SystemExit(__doc__)
    src = os.path.join(argv[1], "tests", "test_causal_conv1d.py")
    if not os.path.isfile(src):
        raise SystemExit(f"not found: {src}")
    os.makedirs(DEST, exist_ok=True)
    dst = os.path.join(DEST, "test_causal_conv1d.py")
    shutil.copyfile(src, dst)
    shutil.copyfile(os.path.join(HERE, "reference_conftest.py"), os.path.join(DEST, "conftest.py"))
    with open(dst, "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    with open(os.path.join(DEST, "SOURCE.txt"), "w") as f:
        f.write(f"tests/test_causal_conv1d.py of the reference project, unmodified\nsha256 {digest}\n")
    print(dst, digest)


if __name__ == "__main__":
    main(sys.argv)
