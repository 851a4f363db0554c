"""Seeded random sweep over shapes, strides, offsets, dtypes and flags for every entry point
against the CPU oracle.  Complements the reference-style grids: odd sizes, tensors that are
slices of wider buffers at odd offsets (aligned and not), tiny problems, ragged tails.
Tolerances: fp32 1e-5, fp16 3e-3, bf16 1e-2 as |a-b| <= tol*max(1,|b|); sums relative to
max|ref|; states bit-exact."""
import random

import pytest
import torch

import oracle
from conftest import TOL, assert_close, assert_close_sum

pytestmark = pytest.mark.gpu

DEV = "cuda"
ITYPES = [torch.float32, torch.float16, torch.bfloat16]
SUM_TOL = {torch.float32: 2e-5, torch.float16: 3e-3, torch.bfloat16: 1e-2}


def _api():
    import causal_conv1d_b200 as m
    return m


def _view(rng, shape, dtype, channel_last, align_elems):
    """A (B, D, L) tensor that is a window of a wider buffer: random padding on every side.
    align_elems > 0 keeps the window's offset and row strides multiples of it."""
    B, D, L = shape
    q = (lambda n: ((n + align_elems - 1) // align_elems) * align_elems) if align_elems else (lambda n: n)
    if channel_last:
        lead, tail = q(rng.randrange(0, 17)), q(rng.randrange(0, 17))
        buf = torch.randn(B, L + rng.randrange(0, 3), lead + D + tail, device=DEV, dtype=dtype)
        return buf[:, :L, lead:lead + D].transpose(1, 2)
    lead, tail = q(rng.randrange(0, 9)), q(rng.randrange(0, 9))
    buf = torch.randn(B, D + rng.randrange(0, 3), lead + L + tail, device=DEV, dtype=dtype)
    return buf[:, :D, lead:lead + L]


@pytest.mark.parametrize("seed", range(60))
def test_fwd_bwd_random(seed):
    rng = random.Random(1000 + seed)
    torch.manual_seed(1000 + seed)
    itype = rng.choice(ITYPES)
    wtype = rng.choice([torch.float32, itype])
    channel_last = rng.random() < 0.5
    W = rng.choice([2, 3, 4])
    B = rng.choice([1, 1, 2, 3])
    L = rng.choice([1, 2, 3, 5, 8, 31, 64, 100, 257, 600, 1030])
    D = rng.choice([8, 16, 40, 264]) if channel_last else rng.choice([1, 3, 8, 37, 130])
    silu, has_bias = rng.random() < 0.7, rng.random() < 0.7
    aligned = channel_last or rng.random() < 0.6           # channel-last requires 8-element alignment
    x = _view(rng, (B, D, L), itype, channel_last, 8 if aligned else 0)
    dout = _view(rng, (B, D, L), itype, channel_last, 8 if aligned else 0)
    w = torch.randn(D, W, device=DEV, dtype=wtype)
    b = torch.randn(D, device=DEV, dtype=wtype) if has_bias else None
    use_seq = channel_last and rng.random() < 0.35
    use_states = channel_last and not use_seq and rng.random() < 0.5
    seq_idx = ini = None
    if use_seq:
        ids, t = [], 0
        while len(ids) < L:
            n = rng.randrange(1, 40)
            ids += [t] * n
            t += 1
        seq_idx = torch.tensor(ids[:L], dtype=torch.int32).repeat(B, 1)
        if rng.random() < 0.5 and L > 3:
            seq_idx[:, L - rng.randrange(1, 4):] = -1      # padded tail
        seq_idx = seq_idx.to(DEV)
    if use_states:
        ini = torch.randn(B, W - 1, D, device=DEV, dtype=itype).transpose(1, 2)
    act = "silu" if silu else None

    xr, wr = x.detach().requires_grad_(), w.detach().requires_grad_()
    br = b.detach().requires_grad_() if b is not None else None
    ir = ini.detach().requires_grad_() if ini is not None else None
    res = _api().causal_conv1d_fn(xr, wr, br, seq_idx=seq_idx, initial_states=ir, return_final_states=use_states,
                                  activation=act)
    out, fs = res if use_states else (res, None)
    dfin = torch.randn_like(fs) if fs is not None else None
    if fs is not None:
        torch.autograd.backward([out, fs], [dout, dfin])
    else:
        out.backward(dout)

    ref = oracle.fwd(x, w, b, seq_idx=seq_idx, initial_states=ini, return_final_states=use_states, activation=act)
    ref_out, ref_fs = ref if use_states else (ref, None)
    tol = max(TOL[itype], TOL[wtype])
    assert_close(out, ref_out.to(itype), tol, "out")
    if fs is not None:
        assert torch.equal(fs.cpu(), ref_fs.to(itype)), "final_states"
    g = oracle.bwd(x, w, b, dout, seq_idx=seq_idx, initial_states=ini, dfinal_states=dfin, activation=act)
    assert_close(xr.grad, g["dx"].to(itype), tol, "dx")
    stol = max(SUM_TOL[itype], TOL[wtype])
    assert_close_sum(wr.grad, g["dweight"].to(wtype), stol, "dweight")
    if b is not None:
        assert_close_sum(br.grad, g["dbias"].to(wtype), stol, "dbias")
    if ini is not None:
        assert_close(ir.grad, g["dinitial_states"].to(itype), tol, "dinitial_states")


@pytest.mark.parametrize("seed", range(40))
def test_update_random(seed):
    rng = random.Random(2000 + seed)
    torch.manual_seed(2000 + seed)
    itype = rng.choice(ITYPES)
    wtype = rng.choice([torch.float32, itype])
    W = rng.choice([2, 3, 4])
    B = rng.choice([1, 2, 5, 9])
    D = rng.choice([1, 8, 24, 100, 264])
    Lx = rng.choice([1, 1, 2, 4, 7])
    circ = rng.random() < 0.4
    S = W - 1 + rng.choice([0, 0, 1, 3, 6])
    if circ and Lx > S:
        S = Lx + rng.randrange(0, 3)       # the circular reference has no defined order when tokens wrap onto each other
    pool = B + rng.randrange(0, 4)
    state_cl, x_cl = rng.random() < 0.5, rng.random() < 0.5
    st = torch.randn(pool, S, D, device=DEV, dtype=itype).transpose(1, 2) if state_cl else torch.randn(pool, D, S, device=DEV, dtype=itype)
    x = torch.randn(B, Lx, D, device=DEV, dtype=itype).transpose(1, 2) if x_cl else torch.randn(B, D, Lx, device=DEV, dtype=itype)
    w = torch.randn(D, W, device=DEV, dtype=wtype)
    b = torch.randn(D, device=DEV, dtype=wtype) if rng.random() < 0.7 else None
    idx = None
    if rng.random() < 0.7:
        idx = torch.randperm(pool)[:B].to(torch.int32)
        if B > 1 and rng.random() < 0.5:
            idx[rng.randrange(B)] = -1
        idx = idx.to(DEV)
    elif pool != B:
        st = st[:B]
    cache = torch.randint(0, 5000, (B,), dtype=torch.int32, device=DEV) if circ else None
    act = "silu" if rng.random() < 0.7 else None
    ref_out, ref_st = oracle.update(x, st, w, b, activation=act, cache_seqlens=cache, conv_state_indices=idx)
    out = _api().causal_conv1d_update(x, st, w, b, activation=act, cache_seqlens=cache, conv_state_indices=idx)
    assert torch.equal(st.cpu(), ref_st.to(itype)), "conv_state must be bit-exact"
    assert_close(out, ref_out.to(itype), max(TOL[itype], TOL[wtype]), "out")


@pytest.mark.parametrize("seed", range(25))
def test_prefill_and_varlen_states_random(seed):
    from causal_conv1d_b200.causal_conv1d_varlen import causal_conv1d_varlen_fn, causal_conv1d_varlen_states
    rng = random.Random(3000 + seed)
    torch.manual_seed(3000 + seed)
    itype = rng.choice(ITYPES)
    W = rng.choice([2, 3, 4])
    D = rng.choice([8, 24, 136, 520])
    nseq = rng.choice([1, 2, 5, 12])
    lens = [rng.choice([0, 1, 2, 3, 9, 40, 130]) for _ in range(nseq)]
    pad = rng.choice([0, 0, 4])
    cu = torch.tensor([0] + lens, dtype=torch.int64).cumsum(0)
    total = int(cu[-1]) + pad
    lead = 8 * rng.randrange(0, 3)
    x = torch.randn(max(total, 1), lead + D + 8, device=DEV, dtype=itype)[:total, lead:lead + D]
    w = torch.randn(D, W, device=DEV)
    b = torch.randn(D, device=DEV) if rng.random() < 0.6 else None
    S = W - 1 + rng.choice([0, 0, 2, 5])
    rows = nseq + rng.randrange(0, 3)
    pool = torch.randn(rows, S, D, device=DEV, dtype=itype).transpose(1, 2)
    idx = torch.randperm(rows)[:nseq].to(torch.int32) if rng.random() < 0.6 else None
    has = (torch.rand(nseq) < 0.5) if rng.random() < 0.6 else None
    act = "silu" if rng.random() < 0.7 else None
    # states of a plain gather first (int64 cu_seqlens, like the reference's test)
    st = causal_conv1d_varlen_states(x, cu.to(DEV), S)
    assert torch.equal(st.cpu(), oracle.varlen_states(x, cu, S).to(itype))
    ref_out, ref_pool = oracle.prefill_varlen(x, w, b, cu, pool, idx, has, activation=act)
    out = causal_conv1d_varlen_fn(x, w, b, cu_seqlens=cu.to(DEV), conv_states=pool,
                                  state_indices=None if idx is None else idx.to(DEV),
                                  has_initial_state=None if has is None else has.to(DEV), activation=act)
    assert_close(out, ref_out.to(itype), TOL[itype], "out")
    assert torch.equal(pool.cpu(), ref_pool.to(itype)), "conv states must be bit-exact"
