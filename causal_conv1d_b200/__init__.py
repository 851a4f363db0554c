"""B200-native (sm_100a) causal depthwise conv1d: a drop-in for the hot path of
Dao-AILab/causal-conv1d.

Same public names and signatures as the reference package (``causal_conv1d/__init__.py:1-3``
and its sub-modules); underneath, hand-written CUDA kernels behind the C ABI of
``include/cc1d.h``.  There is no CPU or Triton fallback: importing the package loads the
native libraries and fails loudly when they cannot be loaded or built.
"""
__version__ = "0.1.0"

from causal_conv1d_b200.causal_conv1d_interface import (  # noqa: F401
    CausalConv1dFn,
    causal_conv1d_fn,
    causal_conv1d_update,
)
from causal_conv1d_b200.causal_conv1d_varlen import causal_conv1d_varlen_states  # noqa: F401


def install_as_causal_conv1d() -> None:
    """Register this package under the reference's module names (``causal_conv1d``,
    ``causal_conv1d.causal_conv1d_interface``, ``causal_conv1d.cpp_functions``,
    ``causal_conv1d.causal_conv1d_varlen``) and the native extension under the name of the
    reference's pybind module (``causal_conv1d_cuda``, ``csrc/causal_conv1d.cpp:559-563``: the
    same three functions with the same positional argument lists) so that unmodified callers
    import it."""
    import sys

    from causal_conv1d_b200 import causal_conv1d_interface, causal_conv1d_varlen, cpp_functions
    from causal_conv1d_b200._ext import ext

    me = sys.modules[__name__]
    sys.modules["causal_conv1d"] = me
    sys.modules["causal_conv1d.causal_conv1d_interface"] = causal_conv1d_interface
    sys.modules["causal_conv1d.cpp_functions"] = cpp_functions
    sys.modules["causal_conv1d.causal_conv1d_varlen"] = causal_conv1d_varlen
    sys.modules["causal_conv1d_cuda"] = ext
