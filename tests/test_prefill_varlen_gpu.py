"""Packed variable-length prefill with per-sequence conv states (cc1d_prefill_varlen /
causal_conv1d_varlen_fn) against the golden fixtures made from the reference's
causal_conv1d_ref per sequence, against the CPU oracle, and against this package's own
per-sequence calls.  Tolerances: fp32 1e-5, fp16 3e-3, bf16 1e-2 as |a-b| <= tol*max(1,|b|);
conv states bit-exact."""
import ctypes

import pytest
import torch

import cabi
import oracle
from conftest import DT, TOL, assert_close, golden_names

pytestmark = pytest.mark.gpu


def _api():
    from causal_conv1d_b200 import causal_conv1d_fn
    from causal_conv1d_b200.causal_conv1d_varlen import (causal_conv1d_varlen_fn, causal_conv1d_varlen_states,
                                                         seq_idx_from_cu_seqlens)
    return causal_conv1d_fn, causal_conv1d_varlen_fn, causal_conv1d_varlen_states, seq_idx_from_cu_seqlens


def _pool(rows, dim, S, dtype):
    """(rows, dim, S) with stride(1) == 1, like the reference's state tensors."""
    return torch.randn(rows, S, dim, device="cuda", dtype=dtype).transpose(1, 2)


@pytest.mark.parametrize("case", golden_names("prefill_varlen"))
def test_golden(golden, case):
    _, varlen_fn, _, _ = _api()
    m = golden.meta[case]
    it = DT[m["itype"]]
    g = lambda k, dt=None: None if golden.get(case, k, dt) is None else golden.get(case, k, dt).cuda()
    pool = g("conv_states", it).transpose(1, 2).contiguous().transpose(1, 2)
    out = varlen_fn(g("x", it), g("weight"), g("bias"), cu_seqlens=g("cu_seqlens"), conv_states=pool,
                    state_indices=g("state_indices"), has_initial_state=g("has_initial_state"),
                    activation="silu" if m["silu"] else None)
    assert_close(out, g("out", it), TOL[it], "out")
    assert torch.equal(pool, g("conv_states_out", it)), "conv states must be bit-exact"


@pytest.mark.parametrize("lens,pad", [([], 0), ([], 40), ([1], 0), ([3, 0, 0, 4], 2), ([0, 5], 0),
                                      ([700, 1, 1, 2048, 0, 13] * 3, 77)])
def test_seq_idx_from_cu_seqlens(lens, pad):
    *_, build = _api()
    cu = torch.tensor([0] + lens, dtype=torch.int64).cumsum(0).to(torch.int32)
    total = int(cu[-1]) + pad
    got = build(cu.cuda(), total).cpu()
    want = torch.full((total,), -1, dtype=torch.int32)
    for s in range(len(lens)):
        want[int(cu[s]):int(cu[s + 1])] = s
    assert torch.equal(got, want)


@pytest.mark.parametrize("itype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("width", [2, 3, 4])
@pytest.mark.parametrize("extra", [0, 3])
def test_against_oracle(itype, width, extra):
    """Sequences that straddle the forward kernel's token boxes and chunks, empty sequences,
    a sequence without a row (negative index), a padded tail, states updated in place."""
    _, varlen_fn, _, _ = _api()
    torch.manual_seed(width * 10 + extra)
    dim, S = 136, width - 1 + extra
    lens = [1, 2, 3, 70, 0, 129, 8, 1, 64, 257, 5]
    nseq = len(lens)
    cu = torch.tensor([0] + lens, dtype=torch.int32).cumsum(0).to(torch.int32)
    total = int(cu[-1]) + 6
    x = torch.randn(total, 200, device="cuda", dtype=itype)[:, 40:40 + dim]       # a slice of a wider projection
    w = torch.randn(dim, width, device="cuda")
    b = torch.randn(dim, device="cuda")
    pool = _pool(nseq + 4, dim, S, itype)
    idx = torch.randperm(nseq + 4)[:nseq].to(torch.int32)
    idx[3] = -1
    has = torch.rand(nseq) < 0.6
    has[0] = has[2] = True
    ref_out, ref_pool = oracle.prefill_varlen(x, w, b, cu, pool, idx, has, activation="silu")
    before = pool.clone()
    out = varlen_fn(x, w, b, cu_seqlens=cu.cuda(), conv_states=pool, state_indices=idx.cuda(),
                    has_initial_state=has.cuda(), activation="silu")
    assert_close(out, ref_out.to(itype), TOL[itype], "out")
    assert (out[int(cu[-1]):] == 0).all(), "tokens after the last sequence output zero"
    assert torch.equal(pool.cpu(), ref_pool.to(itype)), "conv states must be bit-exact"
    free = [r for r in range(nseq + 4) if r not in idx.tolist()]
    assert torch.equal(pool[free], before[free]), "rows no sequence names stay untouched"


@pytest.mark.parametrize("itype", [torch.float32, torch.bfloat16])
def test_equals_per_sequence_calls(itype):
    """The pack gives, bit for bit, what this package's causal_conv1d_fn gives sequence by
    sequence with initial_states / return_final_states, and causal_conv1d_varlen_states when
    nothing is prefixed."""
    conv_fn, varlen_fn, varlen_states, _ = _api()
    torch.manual_seed(5)
    dim, width, S = 256, 4, 3
    lens = [300, 1, 2, 41, 1000, 3]
    cu = torch.tensor([0] + lens, dtype=torch.int32).cumsum(0).to(torch.int32).cuda()
    total = sum(lens)
    x = torch.randn(total, dim, device="cuda", dtype=itype)
    w = torch.randn(dim, width, device="cuda", dtype=itype)
    b = torch.randn(dim, device="cuda", dtype=itype)
    pool = _pool(len(lens), dim, S, itype)
    pool0 = pool.clone()
    out = varlen_fn(x, w, b, cu_seqlens=cu, conv_states=pool, activation="silu")
    for s, n in enumerate(lens):
        beg = int(cu[s])
        xs = x[beg:beg + n].unsqueeze(0).transpose(1, 2)                       # (1, dim, n) channel-last
        o, fs = conv_fn(xs, w, b, initial_states=pool0[s:s + 1], return_final_states=True, activation="silu")
        assert torch.equal(out[beg:beg + n], o[0].T), f"sequence {s}"
        assert torch.equal(pool[s], fs[0]), f"final state of sequence {s}"
    # without a prefix and with a longer state: the gather of causal_conv1d_varlen_states
    big = _pool(len(lens), dim, 7, itype)
    varlen_fn(x, w, b, cu_seqlens=cu, conv_states=big, has_initial_state=torch.zeros(len(lens), dtype=torch.bool, device="cuda"))
    assert torch.equal(big, varlen_states(x, cu, 7))


def test_read_only_and_no_states():
    _, varlen_fn, _, _ = _api()
    torch.manual_seed(9)
    dim, width = 64, 3
    cu = torch.tensor([0, 10, 30], dtype=torch.int32, device="cuda")
    x = torch.randn(30, dim, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(dim, width, device="cuda")
    pool = _pool(2, dim, 2, torch.bfloat16)
    keep = pool.clone()
    out = varlen_fn(x, w, cu_seqlens=cu, conv_states=pool, update_states=False)
    assert torch.equal(pool, keep)
    ref, _ = oracle.prefill_varlen(x, w, None, cu.cpu(), keep)
    assert_close(out, ref.to(torch.bfloat16), TOL[torch.bfloat16], "out")
    out2 = varlen_fn(x, w, cu_seqlens=cu)
    ref2, _ = oracle.prefill_varlen(x, w, None, cu.cpu())
    assert_close(out2, ref2.to(torch.bfloat16), TOL[torch.bfloat16], "out without states")


def test_c_abi_direct_and_errors():
    lib = cabi.load()
    torch.manual_seed(2)
    dim, width, S, total = 64, 4, 3, 50
    cu = torch.tensor([0, 20, 50], dtype=torch.int32, device="cuda")
    x = torch.randn(total, dim, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(x)
    w = torch.randn(dim, width, device="cuda")
    pool = _pool(2, dim, S, torch.bfloat16)
    ref_out, ref_pool = oracle.prefill_varlen(x, w, None, cu.cpu(), pool, activation="silu")
    sidx = torch.empty(total, dtype=torch.int32, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.cc1d_seq_idx_from_cu_seqlens(cu.data_ptr(), 2, total, sidx.data_ptr(), st) == 0
    p = cabi.PrefillParams(itype=cabi.BF16, wtype=cabi.F32, width=width, silu=1, total_tokens=total, dim=dim, nseq=2,
                           state_len=S, x=x.data_ptr(), x_l_stride=dim, weight=w.data_ptr(), weight_c_stride=width,
                           weight_width_stride=1, out=out.data_ptr(), out_l_stride=dim, seq_idx=sidx.data_ptr(),
                           cu_seqlens=cu.data_ptr(), initial_states=pool.data_ptr(),
                           initial_states_batch_stride=pool.stride(0), initial_states_l_stride=pool.stride(2),
                           final_states=pool.data_ptr(), final_states_batch_stride=pool.stride(0),
                           final_states_l_stride=pool.stride(2))
    assert lib.cc1d_prefill_varlen(ctypes.byref(p), st) == 0
    torch.cuda.synchronize()
    assert_close(out, ref_out.to(torch.bfloat16), TOL[torch.bfloat16], "out")
    assert torch.equal(pool.cpu(), ref_pool.to(torch.bfloat16))
    # rejected before any launch
    for field, value, code in (("width", 5, 3), ("state_len", 2, 10), ("dim", 60, 6), ("seq_idx", None, 1),
                               ("initial_states_l_stride", dim + 1, 12)):
        q = cabi.PrefillParams.from_buffer_copy(p)
        setattr(q, field, value)
        assert lib.cc1d_prefill_varlen(ctypes.byref(q), st) == code, field
