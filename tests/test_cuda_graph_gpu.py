"""Every C-ABI entry point is capturable in a CUDA graph (no allocation, no synchronisation,
no host-side state that a replay would miss): capture on a side stream with FRESH shapes —
so that first-call set-up inside the library happens during capture — replay with new input
values in the same buffers and compare with eager calls.  Results must be bit-identical."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _capture(fn):
    g, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    return g


@pytest.mark.parametrize("channel_last", [False, True])
@pytest.mark.parametrize("itype", [torch.float32, torch.bfloat16])
def test_fwd_bwd_in_graph(itype, channel_last):
    from causal_conv1d_b200._ext import ext
    torch.manual_seed(0)
    B, D, L, W = 2, 264, 611 if channel_last else 616, 4      # shapes no other test uses
    mk = (lambda: torch.randn(B, L, D, device="cuda", dtype=itype).transpose(1, 2)) if channel_last else \
         (lambda: torch.randn(B, D, L, device="cuda", dtype=itype))
    x, dout = mk(), mk()
    w, b = torch.randn(D, W, device="cuda"), torch.randn(D, device="cuda")
    out, dx = torch.empty_like(x), torch.empty_like(x)
    dw, db = torch.empty(D, W, device="cuda"), torch.empty(D, device="cuda")
    ini = torch.randn(B, W - 1, D, device="cuda", dtype=itype).transpose(1, 2) if channel_last else None
    fin = torch.empty_like(ini) if channel_last else None
    dini = torch.empty_like(ini) if channel_last else None

    def step():
        ext.causal_conv1d_fwd(x, w, b, None, ini, out, fin, True)
        ext.causal_conv1d_bwd(x, w, b, dout, None, ini, None, dx, dw, db, dini, True, False)

    g = _capture(step)
    x.copy_(mk()); dout.copy_(mk())            # new values, same buffers
    g.replay()
    torch.cuda.synchronize()
    got = [t.clone() for t in (out, dx, dw, db) + ((fin, dini) if channel_last else ())]
    step()
    torch.cuda.synchronize()
    want = (out, dx, dw, db) + ((fin, dini) if channel_last else ())
    assert all(torch.equal(a, c) for a, c in zip(got, want))


def test_update_varlen_prefill_in_graph():
    from causal_conv1d_b200._ext import ext
    torch.manual_seed(1)
    D, W, S = 328, 3, 4
    w, b = torch.randn(D, W, device="cuda"), torch.randn(D, device="cuda")
    bf = torch.bfloat16
    # decode update
    xs = torch.randn(5, D, 1, device="cuda", dtype=bf)
    pool = torch.randn(9, S, D, device="cuda", dtype=bf).transpose(1, 2)
    idx = torch.tensor([3, -1, 0, 8, 5], dtype=torch.int32, device="cuda")
    uo = torch.empty_like(xs)
    # packed prefill with states
    cu = torch.tensor([0, 11, 11, 40, 41], dtype=torch.int32, device="cuda")
    xp = torch.randn(41, D, device="cuda", dtype=bf)
    po, sidx = torch.empty_like(xp), torch.empty(41, dtype=torch.int32, device="cuda")
    ppool = torch.randn(4, S, D, device="cuda", dtype=bf).transpose(1, 2)
    vs = torch.empty(4, S, D, device="cuda", dtype=bf).transpose(1, 2)

    def step():
        ext.causal_conv1d_update(xs, pool, w, b, uo, True, None, idx)
        ext.seq_idx_from_cu_seqlens(cu, sidx)
        ext.causal_conv1d_prefill_varlen(xp, w, b, sidx, cu, ppool, ppool, None, None, po, True)
        ext.causal_conv1d_varlen_states(xp, cu, vs)

    pool0, ppool0 = pool.clone(), ppool.clone()
    g = _capture(step)
    pool.copy_(pool0); ppool.copy_(ppool0)     # capture does not run anything, but be explicit
    xs.copy_(torch.randn_like(xs)); xp.copy_(torch.randn_like(xp))
    g.replay()
    torch.cuda.synchronize()
    got = [t.clone() for t in (uo, pool, po, ppool, vs, sidx)]
    pool.copy_(pool0); ppool.copy_(ppool0)
    step()
    torch.cuda.synchronize()
    assert all(torch.equal(a, c) for a, c in zip(got, (uo, pool, po, ppool, vs, sidx)))
