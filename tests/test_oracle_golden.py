"""The CPU oracle (oracle/) against the fixtures produced by the reference's own PyTorch
functions (tests/golden/make_golden.py).  Runs without a GPU."""
import pytest
import torch

import oracle
from conftest import DT, TOL, assert_close, assert_close_sum, check, golden_names


@pytest.mark.parametrize("case", golden_names("fwd_bwd"))
def test_fwd_bwd(golden, case):
    m = golden.meta[case]
    it, wt = DT[m["itype"]], DT[m["wtype"]]
    g = lambda k, dt: golden.get(case, k, dt)
    x, w, b = g("x", it), g("weight", wt), g("bias", wt)
    ini, dout, dfin = g("initial_states", it), g("dout", it), g("dfinal_states", it)
    act = "silu" if m["silu"] else None
    tol = max(TOL[it], TOL[wt])  # the reference computes in the weight dtype
    res = oracle.fwd(x, w, b, initial_states=ini, return_final_states=m["final"], activation=act)
    out, fs = res if m["final"] else (res, None)
    check(out.to(it), g("out", it), it, wt, "out")
    if m["final"]:
        assert torch.equal(fs.to(it), g("final_states", it)), "final_states must be bit-exact"
    gr = oracle.bwd(x, w, b, dout, initial_states=ini, dfinal_states=dfin, activation=act)
    check(gr["dx"].to(it), g("dx", it), it, wt, "dx")
    assert_close_sum(gr["dweight"], g("dweight", wt), max(tol, 1e-5), "dweight")
    if b is not None:
        assert_close_sum(gr["dbias"], g("dbias", wt), max(tol, 1e-5), "dbias")
    if ini is not None:
        check(gr["dinitial_states"].to(it), g("dinitial_states", it), it, wt, "dinitial_states")


@pytest.mark.parametrize("case", golden_names("seq_idx"))
def test_seq_idx(golden, case):
    m = golden.meta[case]
    it = DT[m["itype"]]
    g = lambda k, dt=None: golden.get(case, k, dt)
    x, w, b, dout, sidx = g("x", it), g("weight"), g("bias"), g("dout", it), g("seq_idx")
    act = "silu" if m["silu"] else None
    out = oracle.fwd(x, w, b, seq_idx=sidx, activation=act)
    assert_close(out.to(it), g("out", it), TOL[it], "out")
    if m["padded"]:
        assert (out[sidx.unsqueeze(1).expand_as(out) < 0] == 0).all()
    gr = oracle.bwd(x, w, b, dout, seq_idx=sidx, activation=act)
    assert_close(gr["dx"].to(it), g("dx", it), TOL[it], "dx")
    assert_close_sum(gr["dweight"], g("dweight"), 1e-5, "dweight")
    if b is not None:
        assert_close_sum(gr["dbias"], g("dbias"), 1e-5, "dbias")


@pytest.mark.parametrize("case", golden_names("update"))
def test_update(golden, case):
    m = golden.meta[case]
    it, wt = DT[m["itype"]], DT[m["wtype"]]
    g = lambda k, dt=None: golden.get(case, k, dt)
    out, st = oracle.update(g("x", it), g("conv_state", it), g("weight", wt), g("bias", wt),
                            activation="silu" if m["silu"] else None, cache_seqlens=g("cache_seqlens"))
    assert torch.equal(st.to(it), g("conv_state_out", it)), "conv_state must be bit-exact"
    check(out.to(it), g("out", it), it, wt, "out")


@pytest.mark.parametrize("case", golden_names("update_gather"))
def test_update_gather(golden, case):
    """conv_state_indices with padded entries: gather -> causal_conv1d_update_ref -> scatter, stored by
    tests/golden/make_golden_gather.py."""
    m = golden.meta[case]
    it, wt = DT[m["itype"]], DT[m["wtype"]]
    g = lambda k, dt=None: golden.get(case, k, dt)
    out, st = oracle.update(g("x", it), g("conv_state", it), g("weight", wt), g("bias", wt),
                            activation="silu" if m["silu"] else None, cache_seqlens=g("cache_seqlens"),
                            conv_state_indices=g("conv_state_indices"))
    assert torch.equal(st.to(it), g("conv_state_out", it)), "pool must be bit-exact"
    idx = g("conv_state_indices")
    assert (out[idx < 0] == 0).all()
    check(out.to(it), g("out", it), it, wt, "out")


@pytest.mark.parametrize("case", golden_names("varlen_states"))
def test_varlen_states(golden, case):
    m = golden.meta[case]
    it = DT[m["itype"]]
    st = oracle.varlen_states(golden.get(case, "x", it), golden.get(case, "cu_seqlens"), m["state_len"])
    assert torch.equal(st.to(it), golden.get(case, "states", it))


@pytest.mark.parametrize("case", golden_names("prefill_varlen"))
def test_prefill_varlen(golden, case):
    """Per-sequence composition of the oracle forward against the per-sequence loop over
    causal_conv1d_ref stored by tests/golden/make_golden_prefill.py."""
    m = golden.meta[case]
    it = DT[m["itype"]]
    g = lambda k, dt=None: golden.get(case, k, dt)
    out, st = oracle.prefill_varlen(g("x", it), g("weight"), g("bias"), g("cu_seqlens"), g("conv_states", it),
                                    g("state_indices"), g("has_initial_state"),
                                    activation="silu" if m["silu"] else None)
    assert_close(out.to(it), g("out", it), TOL[it], "out")
    assert torch.equal(st.to(it), g("conv_states_out", it)), "conv states must be bit-exact"


def test_update_padding_and_gather():
    """Negative conv_state_indices: zero output, pool untouched
    (rule of csrc/causal_conv1d_update.cu:48-54, tested at tests/test_causal_conv1d.py:317-321)."""
    torch.manual_seed(0)
    x = torch.randn(4, 8, 2)
    pool = torch.randn(10, 8, 5)
    w, b = torch.randn(8, 3), torch.randn(8)
    idx = torch.tensor([7, -1, 2, -1], dtype=torch.int32)
    out, st = oracle.update(x, pool, w, b, activation="silu", conv_state_indices=idx)
    assert (out[1] == 0).all() and (out[3] == 0).all()
    untouched = [i for i in range(10) if i not in (7, 2)]
    assert torch.equal(st[untouched], pool[untouched].double())
    out2, st2 = oracle.update(x[[0, 2]], pool[[7, 2]], w, b, activation="silu")
    assert torch.equal(out[[0, 2]], out2) and torch.equal(st[[7, 2]], st2)
