"""Loads the native extension (``_cc1d_torch.so`` -> ``libcc1d.so``).

The libraries are built in-tree by ``causal_conv1d_b200._build``.  When they are missing
and a CUDA toolchain is present they are built on first import; otherwise the import
fails — there is deliberately no fallback implementation.
"""
import importlib
import os

_PKG = os.path.dirname(os.path.abspath(__file__))


def _load():
    try:
        return importlib.import_module("causal_conv1d_b200._cc1d_torch")
    except ImportError as first:
        have = os.path.exists(os.path.join(_PKG, "_cc1d_torch.so"))
        if have:
            raise ImportError(
                "causal_conv1d_b200: the native extension exists but failed to load "
                f"({first}); rebuild with `python -m causal_conv1d_b200._build --force`"
            ) from first
        try:
            from causal_conv1d_b200 import _build

            _build.build()
        except Exception as e:  # no toolchain, compile error ...
            raise ImportError(
                "causal_conv1d_b200: native extension not built and building it failed "
                f"({e}); this package has no CPU or Triton fallback"
            ) from e
        return importlib.import_module("causal_conv1d_b200._cc1d_torch")


ext = _load()
