"""Parity of the CUDA path (Python API -> torch extension -> C ABI -> sm_100a kernels)
against the golden fixtures and the CPU oracle.  The grids follow the reference's own test
file (tests/test_causal_conv1d.py), thinned where the CPU oracle would take too long."""
import itertools
import zlib

import pytest
import torch

import oracle
from conftest import DT, TOL, assert_close, assert_close_sum, check, golden_names
from torch_ref import conv_grads64

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _api():
    import causal_conv1d_b200 as m
    return m


def _pick(key, n):
    """Deterministic pseudo-random choice in range(n) from a test id."""
    return zlib.crc32(repr(key).encode()) % n


# Tolerance for fp32 sums of many terms (dweight/dbias): relative to max |ref|.
SUM_TOL = {torch.float32: 2e-5, torch.float16: 3e-3, torch.bfloat16: 1e-2}


# ------------------------------------------------------------------ golden fixtures
@pytest.mark.parametrize("channel_last", [False, True])
@pytest.mark.parametrize("case", golden_names("fwd_bwd"))
def test_golden_fwd_bwd(golden, case, channel_last):
    m = golden.meta[case]
    if not channel_last and (m["init"] or m["final"]):
        pytest.skip("states need channel-last")
    it, wt = DT[m["itype"]], DT[m["wtype"]]
    g = lambda k, dt: None if golden.get(case, k, dt) is None else golden.get(case, k, dt).to(DEV)
    x, w, b = g("x", it), g("weight", wt), g("bias", wt)
    B, D, L = x.shape
    if channel_last:
        if D % 8:
            pytest.skip("channel-last needs dim % 8 == 0")
        # a slice of a wider token-major buffer, so that stride(2) > 1 even when seqlen == 1
        buf = torch.empty(B, L, D + 8, device=DEV, dtype=it)
        buf[:, :, :D] = x.transpose(1, 2)
        x = buf[:, :, :D].transpose(1, 2)
    ini, dout, dfin = g("initial_states", it), g("dout", it), g("dfinal_states", it)
    if ini is not None:
        ini = ini.transpose(1, 2).contiguous().transpose(1, 2)
    act = "silu" if m["silu"] else None
    x.requires_grad_(); w.requires_grad_()
    if b is not None: b.requires_grad_()
    if ini is not None: ini.requires_grad_()
    res = _api().causal_conv1d_fn(x, w, b, initial_states=ini, return_final_states=m["final"], activation=act)
    out, fs = res if m["final"] else (res, None)
    assert (out.stride(1) == 1) == (x.stride(1) == 1), "out keeps x's layout class"
    check(out, g("out", it), it, wt, "out vs golden")
    if fs is not None:
        assert torch.equal(fs, g("final_states", it)), "final_states must be bit-exact"
        torch.autograd.backward([out, fs], [dout, dfin])
    else:
        out.backward(dout)
    check(x.grad, g("dx", it), it, wt, "dx vs golden")
    assert_close_sum(w.grad, g("dweight", wt), max(SUM_TOL[it], TOL[wt]), "dweight vs golden")
    if b is not None:
        assert_close_sum(b.grad, g("dbias", wt), max(SUM_TOL[it], TOL[wt]), "dbias vs golden")
    if ini is not None:
        check(ini.grad, g("dinitial_states", it), it, wt, "dinitial_states vs golden")
    # tight gate against the float64 oracle, one rounding to the I/O dtype
    xo, wo, bo = x.detach(), w.detach(), None if b is None else b.detach()
    o = oracle.fwd(xo, wo, bo, initial_states=ini, return_final_states=m["final"], activation=act)
    o = o[0] if m["final"] else o
    assert_close(out, o.to(it), TOL[it], "out vs oracle")
    gr = oracle.bwd(xo, wo, bo, dout, initial_states=ini, dfinal_states=dfin, activation=act)
    assert_close(x.grad, gr["dx"].to(it), TOL[it], "dx vs oracle")
    assert_close_sum(w.grad, gr["dweight"].to(wt), max(SUM_TOL[it], TOL[wt]), "dweight vs oracle")


@pytest.mark.parametrize("case", golden_names("seq_idx"))
def test_golden_seq_idx(golden, case):
    m = golden.meta[case]
    it = DT[m["itype"]]
    g = lambda k, dt=None: None if golden.get(case, k, dt) is None else golden.get(case, k, dt).to(DEV)
    x = g("x", it).transpose(1, 2).contiguous().transpose(1, 2).requires_grad_()
    w, b, sidx, dout = g("weight").requires_grad_(), g("bias"), g("seq_idx"), g("dout", it)
    if b is not None: b.requires_grad_()
    out = _api().causal_conv1d_fn(x, w, b, seq_idx=sidx, activation="silu" if m["silu"] else None)
    assert_close(out, g("out", it), TOL[it], "out")
    if m["padded"]:
        assert (out.detach()[(sidx < 0)[:, None, :].expand_as(out)] == 0).all(), "padded tokens must be exactly 0"
    out.backward(dout)
    assert_close(x.grad, g("dx", it), TOL[it], "dx")
    assert_close_sum(w.grad, g("dweight"), SUM_TOL[it], "dweight")
    if b is not None:
        assert_close_sum(b.grad, g("dbias"), SUM_TOL[it], "dbias")


@pytest.mark.parametrize("state_layout", ["channel_last", "channel_first"])
@pytest.mark.parametrize("case", golden_names("update"))
def test_golden_update(golden, case, state_layout):
    m = golden.meta[case]
    it, wt = DT[m["itype"]], DT[m["wtype"]]
    g = lambda k, dt=None: None if golden.get(case, k, dt) is None else golden.get(case, k, dt).to(DEV)
    x, st = g("x", it), g("conv_state", it)
    if state_layout == "channel_last":
        x = x.transpose(1, 2).contiguous().transpose(1, 2)
        st = st.transpose(1, 2).contiguous().transpose(1, 2)
    out = _api().causal_conv1d_update(x, st, g("weight", wt), g("bias", wt),
                                      activation="silu" if m["silu"] else None, cache_seqlens=g("cache_seqlens"))
    assert torch.equal(st, g("conv_state_out", it)), "conv_state must be bit-exact"
    check(out, g("out", it), it, wt, "out")


@pytest.mark.parametrize("state_layout", ["channel_last", "channel_first"])
@pytest.mark.parametrize("case", golden_names("update_gather"))
def test_golden_update_gather(golden, case, state_layout):
    """conv_state_indices (with padded entries) against the fixtures made from the reference's
    causal_conv1d_update_ref by gather / scatter."""
    m = golden.meta[case]
    it, wt = DT[m["itype"]], DT[m["wtype"]]
    g = lambda k, dt=None: None if golden.get(case, k, dt) is None else golden.get(case, k, dt).to(DEV)
    x, pool = g("x", it), g("conv_state", it)
    if state_layout == "channel_last":
        pool = pool.transpose(1, 2).contiguous().transpose(1, 2)
        x = x.transpose(1, 2).contiguous().transpose(1, 2)
    out = _api().causal_conv1d_update(x, pool, g("weight", wt), g("bias", wt), activation="silu" if m["silu"] else None,
                                      cache_seqlens=g("cache_seqlens"), conv_state_indices=g("conv_state_indices"))
    assert torch.equal(pool.cpu(), golden.get(case, "conv_state_out", it)), "pool must be bit-exact"
    idx = g("conv_state_indices")
    assert (out[idx < 0] == 0).all()
    check(out, golden.get(case, "out", it), it, wt, "out")


@pytest.mark.parametrize("case", golden_names("varlen_states"))
def test_golden_varlen_states(golden, case):
    m = golden.meta[case]
    it = DT[m["itype"]]
    x, cu = golden.get(case, "x", it).to(DEV), golden.get(case, "cu_seqlens").to(DEV)
    from causal_conv1d_b200.causal_conv1d_varlen import causal_conv1d_varlen_states
    st = causal_conv1d_varlen_states(x, cu, m["state_len"])
    assert st.stride(1) == 1
    assert torch.equal(st, golden.get(case, "states", it).to(DEV))
    st32 = causal_conv1d_varlen_states(x, cu.int(), m["state_len"])
    assert torch.equal(st32, st)


# ------------------------------------------------------------------ reference-style grids
SEQLENS = [1, 2, 8, 16, 32, 64, 128, 129, 130, 151, 256, 372, 512, 784, 1024, 1134, 2048, 4096]


def _make_x(batch, dim, seqlen, itype, channel_last, pad=64):
    """Non-contiguous slice of a wider tensor, as in tests/test_causal_conv1d.py:84-88."""
    if not channel_last:
        return torch.randn(batch, pad + dim + 64, seqlen, device=DEV, dtype=itype)[:, pad:pad + dim, :]
    return torch.randn(batch, seqlen, pad + dim + 64, device=DEV, dtype=itype)[:, :, pad:pad + dim].transpose(1, 2)


def _run_fwd_bwd(dim, seqlen, width, has_bias, silu, itype, channel_last, init, final, use_cpu_oracle):
    torch.manual_seed(0)
    batch = 2
    x = _make_x(batch, dim, seqlen, itype, channel_last).requires_grad_()
    weight = torch.randn(dim, width, device=DEV, dtype=torch.float32, requires_grad=True)
    bias = torch.randn(dim, device=DEV, dtype=torch.float32, requires_grad=True) if has_bias else None
    ini = (torch.randn(batch, width - 1, dim, device=DEV, dtype=itype).transpose(1, 2).requires_grad_()
           if init else None)
    act = "silu" if silu else None
    res = _api().causal_conv1d_fn(x, weight, bias, initial_states=ini, return_final_states=final, activation=act)
    out, fs = res if final else (res, None)
    dout = torch.randn_like(out)
    dfin = torch.randn(batch, width - 1, dim, device=DEV, dtype=itype).transpose(1, 2) if final else None
    if final:
        torch.autograd.backward([out, fs], [dout, dfin])
    else:
        out.backward(dout)
    if use_cpu_oracle:
        o = oracle.fwd(x, weight, bias, initial_states=ini, return_final_states=final, activation=act)
        o_out, o_fs = o if final else (o, None)
        r = oracle.bwd(x, weight, bias, dout, initial_states=ini, dfinal_states=dfin, activation=act)
        r["out"], r["final_states"] = o_out, o_fs
    else:
        r = conv_grads64(x.detach(), weight.detach(), None if bias is None else bias.detach(), dout,
                         None, None if ini is None else ini.detach(), dfin, act)
        if final is False:
            r["final_states"] = None
    assert_close(out, r["out"].to(itype), TOL[itype], "out")
    if final:
        assert torch.equal(fs.cpu(), r["final_states"].to(itype).cpu()), "final_states must be bit-exact"
    assert_close(x.grad, r["dx"].to(itype), TOL[itype], "dx")
    assert_close_sum(weight.grad, r["dweight"], SUM_TOL[itype], "dweight")
    if has_bias:
        assert_close_sum(bias.grad, r["dbias"], SUM_TOL[itype], "dbias")
    if init:
        assert_close(ini.grad, r["dinitial_states"].to(itype), TOL[itype], "dinitial_states")


@pytest.mark.parametrize("channel_last", [False, True])
@pytest.mark.parametrize("itype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("width", [2, 3, 4])
@pytest.mark.parametrize("seqlen", SEQLENS)
def test_causal_conv1d_small_dim(seqlen, width, itype, channel_last):
    """dim 64, every seqlen of the reference grid; bias / SiLU / states chosen per case."""
    key = (seqlen, width, str(itype), channel_last)
    has_bias, silu = bool(_pick(key + ("b",), 2)), bool(_pick(key + ("s",), 2))
    init = final = False
    if channel_last:
        init, final = bool(_pick(key + ("i",), 2)), bool(_pick(key + ("f",), 2))
    _run_fwd_bwd(64, seqlen, width, has_bias, silu, itype, channel_last, init, final, use_cpu_oracle=True)


@pytest.mark.parametrize("channel_last", [False, True])
@pytest.mark.parametrize("itype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("width", [2, 3, 4])
@pytest.mark.parametrize("seqlen", [1, 2, 129, 151, 512, 1134, 4096])
def test_causal_conv1d_wide_dim(seqlen, width, itype, channel_last):
    """dim 4096 + 32 as in the reference grid, checked against the float64 PyTorch statement."""
    key = (seqlen, width, str(itype), channel_last, "wide")
    has_bias, silu = bool(_pick(key + ("b",), 2)), bool(_pick(key + ("s",), 2))
    init = final = False
    if channel_last:
        init, final = bool(_pick(key + ("i",), 2)), bool(_pick(key + ("f",), 2))
    _run_fwd_bwd(4096 + 32, seqlen, width, has_bias, silu, itype, channel_last, init, final, use_cpu_oracle=False)


@pytest.mark.parametrize("itype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("width", [2, 3, 4])
@pytest.mark.parametrize("silu", [False, True])
@pytest.mark.parametrize("batch,dim,seqlen", [(1, 8, 1024), (2, 24, 2048), (1, 3, 8192), (3, 5, 3072),
                                              (2, 24, 2000), (1, 8, 528), (3, 5, 16), (2, 7, 1040), (1, 3, 8176)])
def test_channel_first_rows_of_whole_groups(batch, dim, seqlen, silu, width, itype):
    """16-bit channel-first rows whose length is a multiple of 16 elements on 32-byte aligned rows take
    the kernels that move 32 bytes per lane (whole 1024-element groups: the variant without bounds
    tests; otherwise lanes past the row end idle); few rows, so that rows are cut into several warp
    units (the seeded right halo).  Checked against the CPU oracle, and bit-for-bit against the same
    problem placed 16 bytes off a 32-byte boundary (which takes the 16-byte kernels)."""
    torch.manual_seed(7)
    x = torch.randn(batch, dim, seqlen, device=DEV, dtype=itype)
    dout = torch.randn_like(x)
    w = torch.randn(dim, width, device=DEV)
    b = torch.randn(dim, device=DEV)
    act = "silu" if silu else None

    def run(xv, dv):
        xr, wr, br = xv.detach().requires_grad_(), w.detach().requires_grad_(), b.detach().requires_grad_()
        out = _api().causal_conv1d_fn(xr, wr, br, activation=act)
        out.backward(dv)
        return out, xr.grad, wr.grad, br.grad

    out, dx, dw, db = run(x, dout)
    r = oracle.bwd(x, w, b, dout, activation=act)
    assert_close(out, oracle.fwd(x, w, b, activation=act).to(itype), TOL[itype], "out")
    assert_close(dx, r["dx"].to(itype), TOL[itype], "dx")
    assert_close_sum(dw, r["dweight"], SUM_TOL[itype], "dweight")
    assert_close_sum(db, r["dbias"], SUM_TOL[itype], "dbias")
    # the same rows at an offset of 8 elements inside rows of seqlen + 16 elements
    shifted = lambda t: torch.cat([t.new_zeros(batch, dim, 8), t, t.new_zeros(batch, dim, 8)], dim=-1)[..., 8:8 + seqlen]
    out2, dx2, dw2, db2 = run(shifted(x), shifted(dout))
    assert torch.equal(out, out2) and torch.equal(dx, dx2)
    assert_close_sum(dw2, dw, 2e-5, "dweight, other kernel")
    assert_close_sum(db2, db, 2e-5, "dbias, other kernel")


@pytest.mark.parametrize("silu,has_bias,init,final", list(itertools.product([False, True], repeat=4)))
@pytest.mark.parametrize("width", [2, 3, 4])
def test_causal_conv1d_all_flag_combos(width, silu, has_bias, init, final):
    """Every bias x SiLU x initial_states x return_final_states combination, channel-last bf16/fp32."""
    for itype, seqlen in ((torch.bfloat16, 151), (torch.float32, 2), (torch.float16, 1)):
        _run_fwd_bwd(72, seqlen, width, has_bias, silu, itype, True, init, final, use_cpu_oracle=True)


def _update_inputs(dim, width, seqlen, itype, entries, batch=64, state_layout="channel_last"):
    torch.manual_seed(0)
    x = torch.randn(batch, seqlen, dim, device=DEV, dtype=itype).transpose(-1, -2)
    state_len = int(torch.randint(width - 1, width + 10, (1,)).item())
    if state_layout == "channel_last":
        st = torch.randn(entries, state_len, dim, device=DEV, dtype=itype).transpose(-1, -2)
    else:
        st = torch.randn(entries, dim, state_len, device=DEV, dtype=itype)
    weight = torch.randn(dim, width, device=DEV, dtype=torch.float32)
    return x, st, weight


@pytest.mark.parametrize("state_layout", ["channel_last", "channel_first"])
@pytest.mark.parametrize("itype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("has_cache_seqlens", [False, True])
@pytest.mark.parametrize("seqlen", [1, 4, 5])
@pytest.mark.parametrize("width", [2, 3, 4])
@pytest.mark.parametrize("dim", [2048, 2048 + 16, 4096])
def test_causal_conv1d_update(dim, width, seqlen, has_cache_seqlens, itype, state_layout):
    key = (dim, width, seqlen, has_cache_seqlens, str(itype), state_layout)
    has_bias, silu = bool(_pick(key + ("b",), 2)), bool(_pick(key + ("s",), 2))
    x, st, weight = _update_inputs(dim, width, seqlen, itype, 64, state_layout=state_layout)
    bias = torch.randn(dim, device=DEV, dtype=torch.float32) if has_bias else None
    cache = torch.randint(0, 1024, (64,), dtype=torch.int32, device=DEV) if has_cache_seqlens else None
    if has_cache_seqlens and seqlen > st.shape[-1]:
        pytest.skip("circular write longer than the buffer is order-dependent in the reference oracle")
    act = "silu" if silu else None
    o_out, o_st = oracle.update(x, st, weight, bias, activation=act, cache_seqlens=cache)
    out = _api().causal_conv1d_update(x, st, weight, bias, activation=act, cache_seqlens=cache)
    assert torch.equal(st.cpu(), o_st.to(itype)), "conv_state must be bit-exact"
    assert_close(out, o_out.to(itype), TOL[itype], "out")
    # 2-D x (batch, dim) path
    if seqlen == 1:
        x2, st2, _ = _update_inputs(dim, width, 1, itype, 64, state_layout=state_layout)
        out2 = _api().causal_conv1d_update(x2.squeeze(-1), st2, weight, bias, activation=act, cache_seqlens=cache)
        assert out2.shape == (64, dim)
        assert torch.equal(out2, out.squeeze(-1)) and torch.equal(st2, st)


@pytest.mark.parametrize("itype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("has_cache_seqlens", [False, True])
@pytest.mark.parametrize("seqlen", [1, 4, 5])
@pytest.mark.parametrize("width", [2, 3, 4])
@pytest.mark.parametrize("dim", [2048 + 16, 4096])
def test_causal_conv1d_update_with_batch_gather(dim, width, seqlen, has_cache_seqlens, itype):
    batch = 64
    x, st, weight = _update_inputs(dim, width, seqlen, itype, 10 * batch)
    bias = torch.randn(dim, device=DEV, dtype=torch.float32)
    idx = torch.randperm(10 * batch)[:batch].to(dtype=torch.int32, device=DEV)
    cache = torch.randint(0, 1024, (batch,), dtype=torch.int32, device=DEV) if has_cache_seqlens else None
    if has_cache_seqlens and seqlen > st.shape[-1]:
        pytest.skip("circular write longer than the buffer is order-dependent in the reference oracle")
    o_out, o_st = oracle.update(x, st, weight, bias, activation="silu", cache_seqlens=cache, conv_state_indices=idx)
    out = _api().causal_conv1d_update(x, st, weight, bias, activation="silu", cache_seqlens=cache,
                                      conv_state_indices=idx)
    assert torch.equal(st.cpu(), o_st.to(itype)), "pool must be bit-exact (gathered rows updated, others untouched)"
    assert_close(out, o_out.to(itype), TOL[itype], "out")


@pytest.mark.parametrize("state_layout", ["channel_last", "channel_first"])
@pytest.mark.parametrize("itype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("seqlen", [1, 4, 5])
@pytest.mark.parametrize("width", [2, 3, 4])
def test_causal_conv1d_update_with_padding(width, seqlen, itype, state_layout):
    batch, dim = 64, 2048 + 16
    x, st, weight = _update_inputs(dim, width, seqlen, itype, 10 * batch, state_layout=state_layout)
    bias = torch.randn(dim, device=DEV, dtype=torch.float32)
    valid = torch.randperm(10 * batch)[:batch // 2].to(DEV)
    idx = torch.cat([valid, torch.full((batch - batch // 2,), -1, device=DEV)])[torch.randperm(batch, device=DEV)].int()
    before = st.clone()
    o_out, o_st = oracle.update(x, st, weight, bias, activation="silu", conv_state_indices=idx)
    out = _api().causal_conv1d_update(x, st, weight, bias, activation="silu", conv_state_indices=idx)
    assert torch.all(out[idx < 0] == 0), "padded rows must output exactly zero"
    assert torch.equal(st.cpu(), o_st.to(itype))
    untouched = torch.ones(10 * batch, dtype=torch.bool, device=DEV)
    untouched[valid] = False
    assert torch.equal(st[untouched], before[untouched])
    assert_close(out, o_out.to(itype), TOL[itype], "out")


@pytest.mark.parametrize("itype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dim", [2048, 2048 + 16, 4096, 100])
def test_causal_conv1d_get_states(dim, itype):
    from causal_conv1d_b200.causal_conv1d_varlen import causal_conv1d_varlen_states
    torch.manual_seed(0)
    seqlens = torch.randint(1, 32, (100,), device=DEV)
    total = int(seqlens.sum())
    x = torch.randn(total, dim, device=DEV, dtype=itype)
    cu = torch.nn.functional.pad(seqlens.cumsum(0), (1, 0))   # int64
    st = causal_conv1d_varlen_states(x, cu, 20)
    assert torch.equal(st.cpu(), oracle.varlen_states(x, cu, 20).to(itype))


@pytest.mark.parametrize("itype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("width", [2, 3, 4])
@pytest.mark.parametrize("seqlen", [8, 16, 32, 64, 128, 151, 256, 372, 512, 784, 1024, 1134, 2048, 4096])
@pytest.mark.parametrize("dim", [64, 4096 + 32])
def test_causal_conv1d_varlen(dim, seqlen, width, itype):
    """seq_idx fwd + bwd (tests/test_causal_conv1d.py:401-472), random sub-sequence splits,
    half of the cases with a padded (-1) tail (:474-557)."""
    key = (dim, seqlen, width, str(itype))
    if dim > 64 and _pick(key, 3):
        pytest.skip("thinned")
    has_bias, silu, padded = bool(_pick(key + ("b",), 2)), bool(_pick(key + ("s",), 2)), bool(_pick(key + ("p",), 2))
    torch.manual_seed(seqlen + dim + width)
    batch = 3
    rows = []
    for b in range(batch):
        true_len = int(torch.randint(seqlen // 2, seqlen, (1,))) if padded else seqlen
        nsplits = int(torch.randint(1, 5, (1,)))
        eos = torch.randperm(true_len - 1)[:nsplits].sort().values if true_len > 1 else torch.tensor([], dtype=torch.long)
        bounds = torch.cat([torch.tensor([-1]), eos, torch.tensor([true_len - 1])])
        lens = torch.diff(bounds).tolist()
        ids = torch.cat([torch.full((int(s),), i + 7 * b, dtype=torch.int32) for i, s in enumerate(lens)])
        rows.append(torch.cat([ids, torch.full((seqlen - true_len,), -1, dtype=torch.int32)]))
    sidx = torch.stack(rows).to(DEV)
    x = _make_x(batch, dim, seqlen, itype, True).requires_grad_()
    weight = torch.randn(dim, width, device=DEV, dtype=torch.float32, requires_grad=True)
    bias = torch.randn(dim, device=DEV, dtype=torch.float32, requires_grad=True) if has_bias else None
    act = "silu" if silu else None
    out = _api().causal_conv1d_fn(x, weight, bias, seq_idx=sidx, activation=act)
    dout = torch.randn_like(out)
    out.backward(dout)
    r = conv_grads64(x.detach(), weight.detach(), None if bias is None else bias.detach(), dout, sidx, None, None, act)
    assert_close(out, r["out"].to(itype), TOL[itype], "out")
    assert (out.detach()[(sidx < 0)[:, None, :].expand_as(out)] == 0).all()
    assert_close(x.grad, r["dx"].to(itype), TOL[itype], "dx")
    assert_close_sum(weight.grad, r["dweight"], SUM_TOL[itype], "dweight")
    if has_bias:
        assert_close_sum(bias.grad, r["dbias"], SUM_TOL[itype], "dbias")
    if dim == 64:   # and the CPU oracle on the small ones
        o = oracle.fwd(x, weight, bias, seq_idx=sidx, activation=act)
        assert_close(out, o.to(itype), TOL[itype], "out vs oracle")


@pytest.mark.parametrize("channel_last", [False, True])
def test_bwd_bitwise_reproducible(channel_last):
    """10 backward runs give identical bits (the reference only promises this in its
    deterministic mode, tests/test_causal_conv1d.py:560-575)."""
    torch.manual_seed(123)
    batch, dim, seqlen, width = 4, 1024, 2048, 4
    if channel_last:
        x = torch.randn(batch, seqlen, dim, device=DEV, dtype=torch.bfloat16).transpose(1, 2).requires_grad_()
    else:
        x = torch.randn(batch, dim, seqlen, device=DEV, dtype=torch.bfloat16).requires_grad_()
    w = torch.randn(dim, width, device=DEV, requires_grad=True)
    b = torch.randn(dim, device=DEV, requires_grad=True)
    g = torch.randn_like(x)
    ref = None
    for _ in range(10):
        x.grad = w.grad = b.grad = None
        _api().causal_conv1d_fn(x, w, b, activation="silu").backward(g)
        cur = (x.grad.clone(), w.grad.clone(), b.grad.clone())
        if ref is None:
            ref = cur
        else:
            assert all(torch.equal(a, c) for a, c in zip(ref, cur))


def test_weight_dtypes_and_strides():
    """16-bit weights (the dtype the reference tests never exercise) and a strided weight view."""
    torch.manual_seed(5)
    for itype, wtype in ((torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16), (torch.float32, torch.bfloat16)):
        x = torch.randn(2, 40, 100, device=DEV, dtype=itype)
        wfull = torch.randn(40, 8, device=DEV).to(wtype)
        w = wfull[:, 1:8:2]   # (40, 4), strides (8, 2)
        b = torch.randn(40, device=DEV).to(wtype)
        out = _api().causal_conv1d_fn(x, w, b, activation="silu")
        assert_close(out, oracle.fwd(x, w, b, activation="silu").to(itype), TOL[itype], "out")


def test_errors():
    api = _api()
    x = torch.randn(2, 16, 32, device=DEV)
    with pytest.raises(RuntimeError, match="width between 2 and 4"):
        api.causal_conv1d_fn(x, torch.randn(16, 5, device=DEV))
    with pytest.raises(NotImplementedError):
        api.causal_conv1d_fn(x, torch.randn(16, 4, device=DEV), activation="relu")
    with pytest.raises(RuntimeError, match="divisible by 8"):
        api.causal_conv1d_fn(torch.randn(2, 32, 12, device=DEV).transpose(1, 2), torch.randn(12, 4, device=DEV))
    with pytest.raises(RuntimeError, match="channel last"):
        api.causal_conv1d_fn(x, torch.randn(16, 4, device=DEV), seq_idx=torch.zeros(2, 32, dtype=torch.int32, device=DEV))
    with pytest.raises(AssertionError):
        api.causal_conv1d_fn(x, torch.randn(16, 4, device=DEV), return_final_states=True)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        api.causal_conv1d_fn(x.cpu(), torch.randn(16, 4))
    with pytest.raises(RuntimeError, match="width - 1"):
        api.causal_conv1d_update(torch.randn(2, 16, device=DEV), torch.randn(2, 16, 2, device=DEV), torch.randn(16, 4, device=DEV))


def test_empty_inputs():
    """Zero-sized batch / seqlen: empty outputs, zero weight gradients, no error."""
    api = _api()
    w = torch.randn(16, 4, device=DEV, requires_grad=True)
    b = torch.randn(16, device=DEV, requires_grad=True)
    for shape in ((0, 16, 32), (2, 16, 0)):
        x = torch.randn(*shape, device=DEV, requires_grad=True)
        out = api.causal_conv1d_fn(x, w, b, activation="silu")
        assert out.shape == x.shape
        w.grad = b.grad = None
        out.backward(torch.empty_like(out))
        assert x.grad.shape == x.shape
        assert (w.grad == 0).all() and (b.grad == 0).all()
    out = api.causal_conv1d_update(torch.randn(0, 16, device=DEV), torch.randn(0, 16, 3, device=DEV), w.detach(), b.detach())
    assert out.shape == (0, 16)


def test_registered_custom_ops():
    """The torch.library ops (the path torch.compile traces) give the same bits as the direct calls."""
    import causal_conv1d_b200.cpp_functions  # noqa: F401  (registers the ops)
    torch.manual_seed(9)
    x = torch.randn(2, 24, 100, device=DEV, dtype=torch.bfloat16)
    w, b = torch.randn(24, 4, device=DEV), torch.randn(24, device=DEV)
    ref = _api().causal_conv1d_fn(x, w, b, activation="silu")
    out = torch.empty_like(x)
    torch.ops.cc1d_b200._causal_conv1d_fwd_cpp(x, w, b, None, None, out, None, True)
    assert torch.equal(out, ref)
    dout = torch.randn_like(x)
    dx, dw, db = torch.empty_like(x), torch.empty(24, 4, device=DEV), torch.empty(24, device=DEV)
    torch.ops.cc1d_b200._causal_conv1d_bwd_cpp(x, w, b, dout, None, None, None, dx, dw, db, None, True)
    xr = x.clone().requires_grad_()
    wr = w.clone().requires_grad_()
    _api().causal_conv1d_fn(xr, wr, b, activation="silu").backward(dout)
    assert torch.equal(dx, xr.grad) and torch.equal(dw, wr.grad)
    st = torch.randn(2, 3, 24, device=DEV, dtype=torch.bfloat16).transpose(1, 2)
    st2 = st.clone()
    o1 = torch.empty(2, 24, 1, device=DEV, dtype=torch.bfloat16)
    torch.ops.cc1d_b200._causal_conv1d_update_cpp(x[:, :, :1].contiguous(), st, w, b, o1, True, None, None)
    o2 = _api().causal_conv1d_update(x[:, :, 0].contiguous(), st2, w, b, activation="silu")
    assert torch.equal(o1.squeeze(-1), o2) and torch.equal(st, st2)


@pytest.mark.parametrize("channel_last", [False, True])
def test_strided_slices_in_and_out(channel_last):
    """The op between two layout ops of a caller: x is a slice of a wider projection output, the
    result goes straight into a slice of the buffer the next op reads (the `out` hook of
    causal_conv1d_fwd_function), dx into a slice of the projection's gradient (the `dx` hook,
    causal_conv1d/cpp_functions.py:125,132 of the reference).  Same bits as with dense tensors."""
    from causal_conv1d_b200.cpp_functions import causal_conv1d_bwd_function, causal_conv1d_fwd_function
    torch.manual_seed(7)
    B, D, L, W = 2, 256, 520, 4
    it = torch.bfloat16
    w, b = torch.randn(D, W, device=DEV, dtype=it), torch.randn(D, device=DEV, dtype=it)
    if channel_last:      # (B, L, 2D + 64) projection output, x = channels [D, 2D)
        proj = torch.randn(B, L, 2 * D + 64, device=DEV, dtype=it)
        nxt, dproj = torch.zeros_like(proj), torch.zeros_like(proj)
        sl = lambda t: t[:, :, D:2 * D].transpose(1, 2)
    else:                 # (B, 2D, L) projection output, x = first half of the channels
        proj = torch.randn(B, 2 * D, L, device=DEV, dtype=it)
        nxt, dproj = torch.zeros_like(proj), torch.zeros_like(proj)
        sl = lambda t: t[:, :D]
    x, dout = sl(proj), sl(torch.randn_like(proj))
    out = causal_conv1d_fwd_function(x, w, b, None, None, None, True, out=sl(nxt))
    assert out.data_ptr() == sl(nxt).data_ptr()
    dense = causal_conv1d_fwd_function(x.contiguous() if not channel_last else x.transpose(1, 2).contiguous().transpose(1, 2),
                                       w, b, None, None, None, True)
    assert torch.equal(out, dense)
    untouched = nxt.clone()
    sl(untouched).zero_()
    assert not untouched.any(), "nothing outside the slice is written"
    dx, dw, db, _ = causal_conv1d_bwd_function(x, w, b, dout, None, None, None, sl(dproj), False, True)
    dx2, dw2, db2, _ = causal_conv1d_bwd_function(x, w, b, dout, None, None, None, None, False, True)
    assert dx.data_ptr() == sl(dproj).data_ptr() and torch.equal(dx, dx2) and torch.equal(dw, dw2) and torch.equal(db, db2)
    ref = oracle.fwd(x, w, b, activation="silu")
    assert_close(out, ref.to(it), TOL[it], "out")


@pytest.mark.parametrize("itype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("mode", ["plain", "seq_idx", "states"])
@pytest.mark.parametrize("batch,dim,seqlen", [(2, 264, 1000), (1, 128, 64), (3, 40, 333), (2, 512, 4096),
                                              (1, 5376, 16384)])   # the last one is large enough for 160-token chunks
def test_channel_first_dout_beside_channel_last_x(batch, dim, seqlen, mode, itype):
    """Autograd may hand the backward a channel-first dout although x (and so out) is channel-last.
    The 16-bit kernels read such a dout where it lies (rows 16-byte aligned: seqlen % 8 == 0), every
    other case goes through one re-layout copy; either way the results are those of a channel-last
    dout with the same values, bit for bit."""
    torch.manual_seed(11)
    width = 4
    x = torch.randn(batch, seqlen, dim, device=DEV, dtype=itype).transpose(1, 2)
    w = torch.randn(dim, width, device=DEV)
    b = torch.randn(dim, device=DEV)
    dout_cf = torch.randn(batch, dim, seqlen, device=DEV, dtype=itype)                  # channel-first values
    dout_cl = dout_cf.transpose(1, 2).contiguous().transpose(1, 2)                       # same values, channel-last
    assert dout_cf.stride(2) == 1 and dout_cl.stride(1) == 1
    sidx = ini = dfin = None
    if mode == "seq_idx":
        cut = seqlen // 3
        sidx = torch.cat([torch.zeros(cut), torch.ones(seqlen - cut)]).int().repeat(batch, 1).to(DEV)
    if mode == "states":
        ini = torch.randn(batch, width - 1, dim, device=DEV, dtype=itype).transpose(1, 2)
        dfin = torch.randn(batch, width - 1, dim, device=DEV, dtype=itype).transpose(1, 2)

    def run(dout):
        from causal_conv1d_b200.cpp_functions import causal_conv1d_bwd_function
        return causal_conv1d_bwd_function(x, w, b, dout, sidx, ini, dfin, None, ini is not None, True)

    want = run(dout_cl)
    got = run(dout_cf)
    for a_, b_, name in zip(got, want, ("dx", "dweight", "dbias", "dinitial_states")):
        if b_ is None:
            assert a_ is None
        else:
            assert torch.equal(a_, b_), name
    assert got[0].stride(1) == 1, "dx keeps x's layout"
    # and through autograd: a consumer that made `out` contiguous hands back a channel-first gradient
    xr = x.detach().requires_grad_()
    out = _api().causal_conv1d_fn(xr, w, b, seq_idx=sidx, activation="silu")
    out.contiguous().backward(dout_cf)
    xr2 = x.detach().requires_grad_()
    _api().causal_conv1d_fn(xr2, w, b, seq_idx=sidx, activation="silu").backward(dout_cl)
    assert torch.equal(xr.grad, xr2.grad)
