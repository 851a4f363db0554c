"""The PyTorch statements the package exports under the reference's names
(causal_conv1d_ref, causal_conv1d_update_ref, causal_conv1d_varlen_states_ref) against the
fixtures produced by the reference's own functions (tests/golden/make_golden.py).  No GPU."""
import pytest
import torch

from causal_conv1d_b200.causal_conv1d_interface import causal_conv1d_ref, causal_conv1d_update_ref
from causal_conv1d_b200.causal_conv1d_varlen import causal_conv1d_varlen_states_ref
from conftest import DT, assert_allclose_ref, golden_names


def _close(a, b, dtype, what):
    # Same operators as the generating functions, so differences are at most the last bits that
    # F.conv1d's padded and unpadded code paths may round differently: the reference tests' gate.
    assert_allclose_ref(a, b, dtype, what)


@pytest.mark.parametrize("case", golden_names("fwd_bwd"))
def test_causal_conv1d_ref(golden, case):
    m = golden.meta[case]
    it, wt = DT[m["itype"]], DT[m["wtype"]]
    g = lambda k, dt: golden.get(case, k, dt)
    x = g("x", it).requires_grad_()
    w = g("weight", wt).requires_grad_()
    b = g("bias", wt)
    if b is not None:
        b.requires_grad_()
    ini = g("initial_states", it)
    if ini is not None:
        ini.requires_grad_()
    worse = wt if wt != torch.float32 else it
    res = causal_conv1d_ref(x, w, b, initial_states=ini, return_final_states=m["final"],
                            activation="silu" if m["silu"] else None)
    out, fs = res if m["final"] else (res, None)
    assert out.dtype == it
    _close(out, g("out", it), worse, "out")
    loss = (out.float() * g("dout", it).float()).sum()
    if m["final"]:
        assert torch.equal(fs, g("final_states", it)), "final_states must be bit-exact"
        dfin = g("dfinal_states", it)
        if dfin is not None:
            loss = loss + (fs.float() * dfin.float()).sum()
    loss.backward()
    _close(x.grad, g("dx", it), worse, "dx")
    scale = max(1.0, g("dweight", wt).abs().max().item())
    assert (w.grad.double() - g("dweight", wt).double()).abs().max().item() <= 2e-2 * scale
    if ini is not None and g("dinitial_states", it) is not None:
        _close(ini.grad, g("dinitial_states", it), worse, "dinitial_states")


@pytest.mark.parametrize("case", golden_names("update"))
def test_causal_conv1d_update_ref(golden, case):
    m = golden.meta[case]
    it, wt = DT[m["itype"]], DT[m["wtype"]]
    g = lambda k, dt=None: golden.get(case, k, dt)
    state = g("conv_state", it).clone()
    out = causal_conv1d_update_ref(g("x", it), state, g("weight", wt), g("bias", wt),
                                   activation="silu" if m["silu"] else None, cache_seqlens=g("cache_seqlens"))
    assert torch.equal(state, g("conv_state_out", it)), "conv_state must be bit-exact"
    _close(out, g("out", it), wt if wt != torch.float32 else it, "out")


@pytest.mark.parametrize("case", golden_names("varlen_states"))
def test_causal_conv1d_varlen_states_ref(golden, case):
    m = golden.meta[case]
    it = DT[m["itype"]]
    st = causal_conv1d_varlen_states_ref(golden.get(case, "x", it), golden.get(case, "cu_seqlens"), m["state_len"])
    assert st.stride(1) == 1
    assert torch.equal(st, golden.get(case, "states", it))


def test_names_the_reference_exports_are_importable():
    import sys

    import causal_conv1d_b200
    saved = {k: sys.modules.get(k) for k in ("causal_conv1d", "causal_conv1d.causal_conv1d_interface",
                                             "causal_conv1d.causal_conv1d_varlen", "causal_conv1d.cpp_functions",
                                             "causal_conv1d_cuda")}
    try:
        causal_conv1d_b200.install_as_causal_conv1d()
        from causal_conv1d.causal_conv1d_interface import (  # noqa: F401
            causal_conv1d_fn, causal_conv1d_ref, causal_conv1d_update, causal_conv1d_update_ref)
        from causal_conv1d.causal_conv1d_varlen import (  # noqa: F401
            causal_conv1d_varlen_states, causal_conv1d_varlen_states_ref)
        import causal_conv1d_cuda
        for name in ("causal_conv1d_fwd", "causal_conv1d_bwd", "causal_conv1d_update"):
            assert callable(getattr(causal_conv1d_cuda, name))
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
