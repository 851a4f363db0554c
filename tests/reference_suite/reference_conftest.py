"""conftest.py for a copy of the reference project's own test file.

``prepare.py`` places this file (as ``conftest.py``) next to the copied
``test_causal_conv1d.py``.  It makes ``import causal_conv1d...`` and ``import
causal_conv1d_cuda`` resolve to this repository's package, so the reference's tests run
unmodified against the sm_100a kernels.
"""
import os
import sys

# <repo>/baseline/_ref/reference_tests/conftest.py -> <repo>
_REPO = os.environ.get("CC1D_REPO_ROOT") or os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", ".."))
if _REPO not in sys.path:
    sys.path.insert(0, _REPO)

import causal_conv1d_b200  # noqa: E402

causal_conv1d_b200.install_as_causal_conv1d()
