import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
# Tolerances of the build contract: |a - b| <= tol * max(1, |b|).
TOL = {torch.float32: 1e-5, torch.float16: 3e-3, torch.bfloat16: 1e-2}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def no_kernel_gave_up_waiting():
    """After the last test of a GPU session: no kernel of the library ran out of a bounded wait."""
    yield
    if torch.cuda.is_available():
        from causal_conv1d_b200._ext import ext
        assert ext.wait_expired() == 0, "a TMA kernel gave up a bounded barrier wait during this session"


def assert_close(actual, expected, tol, what=""):
    """|a - b| <= tol * max(1, |b|) elementwise, compared in float64."""
    a = actual.detach().double().cpu()
    b = expected.detach().double().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    if a.numel() == 0:
        return
    err = (a - b).abs() / b.abs().clamp(min=1.0)
    worst = err.max().item()
    assert worst <= tol, f"{what}: max scaled error {worst:.3e} > {tol:.1e}"


def assert_close_sum(actual, expected, tol, what=""):
    """For long reductions (dweight, dbias): error relative to the largest expected entry."""
    a = actual.detach().double().cpu()
    b = expected.detach().double().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    scale = max(1.0, b.abs().max().item())
    worst = (a - b).abs().max().item() / scale
    assert worst <= tol, f"{what}: max error / max|ref| = {worst:.3e} > {tol:.1e}"


# Tolerances the reference's own tests use (tests/test_causal_conv1d.py:75-78): the outer
# gate, applied where the reference oracle itself computes in a 16-bit dtype (16-bit
# weights) and therefore rounds several times.
REF_RTOL_ATOL = {torch.float32: (3e-4, 1e-3), torch.float16: (3e-3, 5e-3), torch.bfloat16: (1e-2, 5e-2)}


def assert_allclose_ref(actual, expected, dtype, what=""):
    rtol, atol = REF_RTOL_ATOL[dtype]
    a = actual.detach().double().cpu()
    b = expected.detach().double().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    bad = (a - b).abs() > atol + rtol * b.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())} elements outside rtol={rtol}, atol={atol}"


def check(actual, expected, itype, wtype, what=""):
    """Tight gate when the reference computed in fp32, the reference tests' gate otherwise."""
    if wtype == torch.float32:
        assert_close(actual, expected, TOL[itype], what)
    else:
        worse = wtype if TOL[wtype] >= TOL[itype] else itype
        assert_allclose_ref(actual, expected, worse, what)


class Golden:
    def __init__(self):
        d = os.path.join(ROOT, "tests", "golden")
        self.arrays, self.meta = {}, {}
        for stem in ("golden", "golden_prefill", "golden_gather"):      # one file per generating script
            self.arrays.update(np.load(os.path.join(d, stem + ".npz")))
            with open(os.path.join(d, stem + ".json")) as f:
                self.meta.update(json.load(f)["cases"])

    def names(self, kind):
        return sorted(n for n, m in self.meta.items() if m["kind"] == kind)

    def get(self, case, key, dtype=None):
        k = f"{case}/{key}"
        if k not in self.arrays:
            return None
        t = torch.from_numpy(self.arrays[k])
        return t.to(dtype) if dtype is not None and t.is_floating_point() else t


_GOLDEN = Golden()


@pytest.fixture(scope="session")
def golden():
    return _GOLDEN


def golden_names(kind):
    return _GOLDEN.names(kind)
