"""Parity at the full sizes of the benchmark configurations (Mamba-1 prefill, packed varlen
prefill, decode update, the 2^31-element stress shape).  The CPU oracle is too slow at these
sizes, so the check is the float64 PyTorch statement of the op (tests/torch_ref.py, itself
checked against the oracle on CPU), evaluated on the GPU — in batch slices where a whole
tensor in float64 would not fit comfortably — plus bit-exact state and determinism checks."""
import pytest
import torch

import oracle
from conftest import TOL, assert_close, assert_close_sum
from torch_ref import conv_grads64

pytestmark = pytest.mark.gpu
DEV = "cuda"
bf16 = torch.bfloat16


def _fn():
    from causal_conv1d_b200 import causal_conv1d_fn
    return causal_conv1d_fn


def _uniform(shape, dtype, gen_seed):
    g = torch.Generator(device="cpu").manual_seed(gen_seed)
    return (torch.rand(*shape, generator=g) - 0.5).to(device=DEV, dtype=dtype)


def test_c2_mamba1_prefill_bf16_channel_first():
    """x (8,5120,2048) bf16 contiguous, weight/bias bf16, SiLU, seed 1: out, dx, dweight, dbias."""
    torch.manual_seed(1)
    x = torch.randn(8, 5120, 2048, device=DEV, dtype=bf16).requires_grad_()
    w = _uniform((5120, 4), bf16, 1).requires_grad_()
    b = _uniform((5120,), bf16, 2).requires_grad_()
    dout = torch.randn(8, 5120, 2048, device=DEV, dtype=bf16)
    out = _fn()(x, w, b, activation="silu")
    out.backward(dout)
    dw_ref = torch.zeros(5120, 4, device=DEV, dtype=torch.float64)
    db_ref = torch.zeros(5120, device=DEV, dtype=torch.float64)
    for i in range(8):   # batch slices keep the float64 graph small
        r = conv_grads64(x.detach()[i:i + 1], w.detach(), b.detach(), dout[i:i + 1], activation="silu")
        assert_close(out[i:i + 1], r["out"].to(bf16), TOL[bf16], f"out[{i}]")
        assert_close(x.grad[i:i + 1], r["dx"].to(bf16), TOL[bf16], f"dx[{i}]")
        dw_ref += r["dweight"]
        db_ref += r["dbias"]
    # gradients are summed in fp32 and rounded once to the bf16 weight dtype
    assert_close_sum(w.grad, dw_ref.to(bf16), 1e-2, "dweight")
    assert_close_sum(b.grad, db_ref.to(bf16), 1e-2, "dbias")


def _packed_lengths(total, n, lo, hi, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n,), generator=g).double()
    lens = (lens / lens.sum() * total).long()
    lens[-1] = total - lens[:-1].sum()
    assert (lens > 0).all()
    return lens


def test_c3a_packed_varlen_seq_idx():
    """bf16 (1,5376,32768) channel-last, 16 packed sequences, seq_idx: fwd + bwd."""
    torch.manual_seed(2)
    L, D = 32768, 5376
    lens = _packed_lengths(L, 16, 256, 3840, 2)
    sidx = torch.repeat_interleave(torch.arange(16), lens).int().view(1, L).to(DEV)
    x = torch.randn(1, L, D, device=DEV, dtype=bf16).transpose(1, 2).requires_grad_()
    w = _uniform((D, 4), bf16, 3).requires_grad_()
    b = _uniform((D,), bf16, 4).requires_grad_()
    dout = torch.randn(1, L, D, device=DEV, dtype=bf16).transpose(1, 2)
    out = _fn()(x, w, b, seq_idx=sidx, activation="silu")
    out.backward(dout)
    dw_ref = torch.zeros(D, 4, device=DEV, dtype=torch.float64)
    db_ref = torch.zeros(D, device=DEV, dtype=torch.float64)
    for c0 in range(0, D, 1344):   # channel slices (channels are independent)
        sl = slice(c0, c0 + 1344)
        r = conv_grads64(x.detach()[:, sl], w.detach()[sl], b.detach()[sl], dout[:, sl], sidx, activation="silu")
        assert_close(out[:, sl], r["out"].to(bf16), TOL[bf16], "out")
        assert_close(x.grad[:, sl], r["dx"].to(bf16), TOL[bf16], "dx")
        dw_ref[sl] = r["dweight"]
        db_ref[sl] = r["dbias"]
    assert_close_sum(w.grad, dw_ref.to(bf16), 1e-2, "dweight")
    assert_close_sum(b.grad, db_ref.to(bf16), 1e-2, "dbias")
    # a sequence never sees its predecessor: zeroing everything before a boundary leaves the
    # outputs after it bit-identical
    cut = int(lens[:5].sum())
    x2 = x.detach().clone()
    x2[:, :, :cut] = 0
    out2 = _fn()(x2, w.detach(), b.detach(), seq_idx=sidx, activation="silu")
    assert torch.equal(out2[:, :, cut:], out.detach()[:, :, cut:])


def test_c3b_states_and_c3c_varlen_states():
    """initial_states / final_states / dinitial_states / dfinal_states at the C3 shape, and
    causal_conv1d_varlen_states on the same packed tokens."""
    from causal_conv1d_b200 import causal_conv1d_varlen_states
    torch.manual_seed(2)
    L, D, W = 32768, 5376, 4
    x = torch.randn(1, L, D, device=DEV, dtype=bf16).transpose(1, 2).requires_grad_()
    w = _uniform((D, W), bf16, 3).requires_grad_()
    b = _uniform((D,), bf16, 4).requires_grad_()
    ini = torch.randn(1, W - 1, D, device=DEV, dtype=bf16).transpose(1, 2).requires_grad_()
    dout = torch.randn(1, L, D, device=DEV, dtype=bf16).transpose(1, 2)
    dfin = torch.randn(1, W - 1, D, device=DEV, dtype=bf16).transpose(1, 2)
    out, fs = _fn()(x, w, b, initial_states=ini, return_final_states=True, activation="silu")
    assert torch.equal(fs, x.detach()[:, :, -(W - 1):]), "final_states = last width-1 tokens, bit-exact"
    torch.autograd.backward([out, fs], [dout, dfin])
    sl = slice(0, 1024)   # a channel slice is enough for the float64 statement
    r = conv_grads64(x.detach()[:, sl], w.detach()[sl], b.detach()[sl], dout[:, sl], None, ini.detach()[:, sl],
                     dfin[:, sl], "silu")
    assert_close(out[:, sl], r["out"].to(bf16), TOL[bf16], "out")
    assert_close(x.grad[:, sl], r["dx"].to(bf16), TOL[bf16], "dx")
    assert_close(ini.grad[:, sl], r["dinitial_states"].to(bf16), TOL[bf16], "dinitial_states")
    assert_close_sum(w.grad[sl], r["dweight"].to(bf16), 1e-2, "dweight")
    # varlen states: (16, 5376, 4) from the packed tokens, int32 cu_seqlens
    lens = _packed_lengths(L, 16, 256, 3840, 2)
    cu = torch.nn.functional.pad(lens.cumsum(0), (1, 0)).int().to(DEV)
    tok = x.detach()[0].transpose(0, 1)   # (32768, 5376) view, channel stride 1
    st = causal_conv1d_varlen_states(tok, cu, 4)
    assert st.shape == (16, D, 4)
    assert torch.equal(st.cpu(), oracle.varlen_states(tok, cu, 4).to(bf16))


@pytest.mark.parametrize("state_layout", ["channel_last", "contiguous"])
@pytest.mark.parametrize("seqlen,circular", [(1, False), (4, False), (1, True), (4, True)])
def test_c4_decode_update(seqlen, circular, state_layout):
    """bf16 x (256,5376,seqlen), pool (512,5376,3) [linear] / (512,5376,8) [circular], indices =
    256 of randperm(512): out close, the whole pool bit-exact."""
    from causal_conv1d_b200 import causal_conv1d_update
    torch.manual_seed(3)
    B, D, W = 256, 5376, 4
    S = 8 if circular else 3
    x = torch.randn(B, D, seqlen, device=DEV, dtype=bf16)
    pool = torch.randn(512, S, D, device=DEV, dtype=bf16).transpose(1, 2) if state_layout == "channel_last" \
        else torch.randn(512, D, S, device=DEV, dtype=bf16)
    w, b = _uniform((D, W), bf16, 5), _uniform((D,), bf16, 6)
    idx = torch.randperm(512)[:B].int().to(DEV)
    cache = torch.randint(0, 10000, (B,), dtype=torch.int32, device=DEV) if circular else None
    o_out, o_pool = oracle.update(x, pool, w, b, activation="silu", cache_seqlens=cache, conv_state_indices=idx)
    out = causal_conv1d_update(x, pool, w, b, activation="silu", cache_seqlens=cache, conv_state_indices=idx)
    assert torch.equal(pool.cpu(), o_pool.to(bf16)), "pool must be bit-exact"
    assert_close(out, o_out.to(bf16), TOL[bf16], "out")


@pytest.mark.parametrize("channel_last", [False, True])
def test_c5_stress_shape_bf16(channel_last):
    """x (32,8192,8192) bf16 = 2^31 elements, width 4, SiLU: out/dx against the float64
    statement on batch slices, dweight/dbias over all slices, 10 backward runs bit-identical."""
    torch.manual_seed(4)
    B, D, L, W = 32, 8192, 8192, 4
    if channel_last:
        x = torch.randn(B, L, D, device=DEV, dtype=bf16).transpose(1, 2)
        dout = torch.randn(B, L, D, device=DEV, dtype=bf16).transpose(1, 2)
    else:
        x = torch.randn(B, D, L, device=DEV, dtype=bf16)
        dout = torch.randn(B, D, L, device=DEV, dtype=bf16)
    x.requires_grad_()
    w = _uniform((D, W), torch.float32, 7).requires_grad_()
    b = _uniform((D,), torch.float32, 8).requires_grad_()
    out = _fn()(x, w, b, activation="silu")
    out.backward(dout)
    dx, dw, db = x.grad, w.grad.clone(), b.grad.clone()
    dw_ref = torch.zeros(D, W, device=DEV, dtype=torch.float64)
    db_ref = torch.zeros(D, device=DEV, dtype=torch.float64)
    for i in range(B):
        r = conv_grads64(x.detach()[i:i + 1], w.detach(), b.detach(), dout[i:i + 1], activation="silu")
        if i % 8 == 0:   # elementwise checks on every 8th slice, the sums over all of them
            assert_close(out[i:i + 1], r["out"].to(bf16), TOL[bf16], f"out[{i}]")
            assert_close(dx[i:i + 1], r["dx"].to(bf16), TOL[bf16], f"dx[{i}]")
        dw_ref += r["dweight"]
        db_ref += r["dbias"]
        del r
    assert_close_sum(dw, dw_ref, 1e-3, "dweight (262144 terms per entry, fp32 accumulation)")
    assert_close_sum(db, db_ref, 1e-3, "dbias")
    del dw_ref, db_ref
    for _ in range(9):
        x.grad = w.grad = b.grad = None
        _fn()(x, w, b, activation="silu").backward(dout)
        assert torch.equal(w.grad, dw) and torch.equal(b.grad, db), "dweight/dbias must be bitwise reproducible"
    assert torch.equal(x.grad, dx)


def test_c5_fp32_and_fp16_reduced_batch():
    """The other dtypes of the stress sweep at batch 4 (fp32 at full batch would need > 40 GB
    with its float64 check): widths 2 and 3, both layouts, with final states on channel-last."""
    torch.manual_seed(4)
    B, D, L = 4, 8192, 8192
    for itype, width, channel_last, silu in ((torch.float32, 3, False, True), (torch.float16, 2, True, False),
                                              (torch.float32, 2, True, True), (torch.float16, 3, False, True)):
        if channel_last:
            x = torch.randn(B, L, D, device=DEV, dtype=itype).transpose(1, 2)
            dout = torch.randn(B, L, D, device=DEV, dtype=itype).transpose(1, 2)
        else:
            x = torch.randn(B, D, L, device=DEV, dtype=itype)
            dout = torch.randn(B, D, L, device=DEV, dtype=itype)
        x.requires_grad_()
        w = _uniform((D, width), torch.float32, 9).requires_grad_()
        b = _uniform((D,), torch.float32, 10).requires_grad_()
        act = "silu" if silu else None
        if channel_last:
            out, fs = _fn()(x, w, b, return_final_states=True, activation=act)
            dfin = torch.randn(B, width - 1, D, device=DEV, dtype=itype).transpose(1, 2)
            assert torch.equal(fs, x.detach()[:, :, -(width - 1):])
            torch.autograd.backward([out, fs], [dout, dfin])
        else:
            out = _fn()(x, w, b, activation=act)
            dfin = None
            out.backward(dout)
        dw_ref = torch.zeros(D, width, device=DEV, dtype=torch.float64)
        for i in range(B):
            r = conv_grads64(x.detach()[i:i + 1], w.detach(), b.detach(), dout[i:i + 1], None, None,
                             None if dfin is None else dfin[i:i + 1], act)
            assert_close(out[i:i + 1], r["out"].to(itype), TOL[itype], f"out[{i}] {itype}")
            assert_close(x.grad[i:i + 1], r["dx"].to(itype), TOL[itype], f"dx[{i}] {itype}")
            dw_ref += r["dweight"]
        assert_close_sum(w.grad, dw_ref, 2e-5 if itype == torch.float32 else 3e-3, f"dweight {itype}")
        del x, dout, out, dw_ref
        torch.cuda.empty_cache()


# The stress sweep at FULL size (batch 32) for the dtype / width / activation / layout combinations
# beyond the two bf16 width-4 cases above: fp32 in both layouts (2^31 elements of 4 bytes: byte offsets
# beyond 2^33), widths 2 and 3 and no activation for each 16-bit dtype.  Channel-last cases run with
# return_final_states and a non-zero dfinal_states.
@pytest.mark.parametrize("itype,width,channel_last,silu", [
    (torch.float32, 4, False, True),
    (torch.float32, 3, True, False),
    (torch.float16, 2, False, False),
    (torch.float16, 3, True, True),
    (torch.bfloat16, 3, False, True),
    (torch.bfloat16, 2, True, False),
])
def test_c5_stress_sweep_full_size(itype, width, channel_last, silu):
    torch.manual_seed(4)
    B, D, L = 32, 8192, 8192
    act = "silu" if silu else None
    if channel_last:
        x = torch.randn(B, L, D, device=DEV, dtype=itype).transpose(1, 2)
        dout = torch.randn(B, L, D, device=DEV, dtype=itype).transpose(1, 2)
        dfin = torch.randn(B, width - 1, D, device=DEV, dtype=itype).transpose(1, 2)
    else:
        x = torch.randn(B, D, L, device=DEV, dtype=itype)
        dout = torch.randn(B, D, L, device=DEV, dtype=itype)
        dfin = None
    x.requires_grad_()
    w = _uniform((D, width), torch.float32, 11).requires_grad_()
    b = _uniform((D,), torch.float32, 12).requires_grad_()

    def run():
        x.grad = w.grad = b.grad = None
        if channel_last:
            out, fs = _fn()(x, w, b, return_final_states=True, activation=act)
            torch.autograd.backward([out, fs], [dout, dfin])
            return out, fs
        out = _fn()(x, w, b, activation=act)
        out.backward(dout)
        return out, None

    out, fs = run()
    if channel_last:
        assert torch.equal(fs, x.detach()[:, :, -(width - 1):]), "final_states must be the last width-1 inputs, bit-exact"
    dx, dw, db = x.grad, w.grad.clone(), b.grad.clone()
    dw_ref = torch.zeros(D, width, device=DEV, dtype=torch.float64)
    db_ref = torch.zeros(D, device=DEV, dtype=torch.float64)
    for i in range(B):
        r = conv_grads64(x.detach()[i:i + 1], w.detach(), b.detach(), dout[i:i + 1], None, None,
                         None if dfin is None else dfin[i:i + 1], act)
        if i % 8 == 0 or i == B - 1:   # elementwise checks on some slices (the last one holds the largest offsets)
            assert_close(out[i:i + 1], r["out"].to(itype), TOL[itype], f"out[{i}]")
            assert_close(dx[i:i + 1], r["dx"].to(itype), TOL[itype], f"dx[{i}]")
        dw_ref += r["dweight"]
        db_ref += r["dbias"]
        del r
    sum_tol = 2e-5 if itype == torch.float32 else 1e-3
    assert_close_sum(dw, dw_ref, sum_tol, "dweight (262144 terms per entry)")
    assert_close_sum(db, db_ref, sum_tol, "dbias")
    del dw_ref, db_ref, out
    for _ in range(9):      # 10 backward runs in all: dweight / dbias / dx bitwise reproducible
        run()
        assert torch.equal(w.grad, dw) and torch.equal(b.grad, db), "dweight/dbias must be bitwise reproducible"
    assert torch.equal(x.grad, dx)
    del x, dout, dx
    torch.cuda.empty_cache()
