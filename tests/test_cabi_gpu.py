"""libcc1d.so driven directly through ctypes with raw device pointers (no torch extension):
what a non-PyTorch host would do."""
import ctypes

import pytest
import torch

import cabi
import oracle
from conftest import TOL, assert_close, assert_close_sum

pytestmark = pytest.mark.gpu
CODE = {torch.float32: cabi.F32, torch.float16: cabi.F16, torch.bfloat16: cabi.BF16}


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("itype", [torch.float32, torch.bfloat16])
def test_fwd_bwd_channel_first_raw(itype):
    lib = cabi.load()
    torch.manual_seed(1)
    B, D, L, W = 3, 40, 264, 4
    x = torch.randn(B, D, L, device="cuda", dtype=itype)
    w = torch.randn(D, W, device="cuda")
    b = torch.randn(D, device="cuda")
    dout = torch.randn_like(x)
    out, dx = torch.empty_like(x), torch.empty_like(x)
    dw, db = torch.full((D, W), 7.0, device="cuda"), torch.full((D,), 7.0, device="cuda")
    fp = cabi.FwdParams(itype=CODE[itype], wtype=cabi.F32, width=W, silu=1, batch=B, dim=D, seqlen=L,
                        x=x.data_ptr(), x_batch_stride=D * L, x_c_stride=L, x_l_stride=1,
                        weight=w.data_ptr(), weight_c_stride=W, weight_width_stride=1, bias=b.data_ptr(),
                        out=out.data_ptr(), out_batch_stride=D * L, out_c_stride=L, out_l_stride=1)
    assert lib.cc1d_fwd(ctypes.byref(fp), _stream()) == 0
    bp = cabi.BwdParams(itype=CODE[itype], wtype=cabi.F32, width=W, silu=1, batch=B, dim=D, seqlen=L,
                        x=x.data_ptr(), x_batch_stride=D * L, x_c_stride=L, x_l_stride=1,
                        weight=w.data_ptr(), weight_c_stride=W, weight_width_stride=1, bias=b.data_ptr(),
                        dout=dout.data_ptr(), dout_batch_stride=D * L, dout_c_stride=L, dout_l_stride=1,
                        dx=dx.data_ptr(), dx_batch_stride=D * L, dx_c_stride=L, dx_l_stride=1,
                        dweight=dw.data_ptr(), dweight_c_stride=W, dweight_width_stride=1, dbias=db.data_ptr(),
                        accumulate=0)
    n = lib.cc1d_bwd_workspace_bytes(ctypes.byref(bp))
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    bp.workspace, bp.workspace_bytes = ws.data_ptr(), n
    assert lib.cc1d_bwd(ctypes.byref(bp), _stream()) == 0
    torch.cuda.synchronize()
    assert_close(out, oracle.fwd(x, w, b, activation="silu").to(itype), TOL[itype], "out")
    g = oracle.bwd(x, w, b, dout, activation="silu")
    assert_close(dx, g["dx"].to(itype), TOL[itype], "dx")
    assert_close_sum(dw, g["dweight"], 2e-5 if itype == torch.float32 else 1e-2, "dweight (overwrite mode)")
    assert_close_sum(db, g["dbias"], 2e-5 if itype == torch.float32 else 1e-2, "dbias (overwrite mode)")
    # accumulate mode adds to what is there (the reference's zero-filled-buffer contract)
    bp.accumulate = 1
    before = dw.clone()
    assert lib.cc1d_bwd(ctypes.byref(bp), _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(dw, before + before)


def test_update_raw_channel_last_state():
    lib = cabi.load()
    torch.manual_seed(2)
    B, D, S, W = 5, 64, 3, 4
    x = torch.randn(B, D, device="cuda", dtype=torch.bfloat16)
    st = torch.randn(B, S, D, device="cuda", dtype=torch.bfloat16)      # memory (B, S, D)
    w = torch.randn(D, W, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(x)
    o_out, o_st = oracle.update(x, st.transpose(1, 2), w, None, activation=None)
    p = cabi.UpdateParams(itype=cabi.BF16, wtype=cabi.BF16, width=W, silu=0, batch=B, dim=D, seqlen=1,
                          x=x.data_ptr(), x_batch_stride=D, x_c_stride=1, x_l_stride=1,
                          weight=w.data_ptr(), weight_c_stride=W, weight_width_stride=1,
                          out=out.data_ptr(), out_batch_stride=D, out_c_stride=1, out_l_stride=1,
                          conv_state=st.data_ptr(), conv_state_len=S,
                          conv_state_batch_stride=S * D, conv_state_c_stride=1, conv_state_l_stride=D)
    assert lib.cc1d_update(ctypes.byref(p), _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(st.transpose(1, 2).cpu(), o_st.to(torch.bfloat16))
    assert_close(out, o_out.to(torch.bfloat16), 1e-2, "out")
