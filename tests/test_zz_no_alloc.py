"""cc1d_bwd_noalloc: the backward for hosts that cannot allocate device memory.

Some callers of libcc1d.so own no allocator they may call at launch time (a plugin whose
host manages all device memory, a latency-critical loop that must never reach cudaMalloc).
cc1d_bwd needs a caller-provided workspace; cc1d_bwd_noalloc does the same work with the
scratch taken from a fixed buffer inside the library (CC1D_NOALLOC_SCRATCH_BYTES = 8 MiB),
so the caller passes inputs and outputs only.

This test drives both entry points through the C ABI on the same inputs, twice in a row
(the shared buffer keeps the first call's contents; the second call must not be disturbed
by them), and checks that the results agree.  It lives in a file that sorts last so that a
run stopping at the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

import cabi
from conftest import TOL, assert_close, assert_close_sum

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 8 * 1024 * 1024
CODE = {torch.float32: cabi.F32, torch.bfloat16: cabi.BF16}


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _params(x, w, b, dout, dx, dw, db, channel_last):
    B, D, L = x.shape
    W = w.shape[1]
    s = lambda t: dict(zip(("batch", "c", "l"), t.stride()))
    p = cabi.BwdParams(itype=CODE[x.dtype], wtype=cabi.F32, width=W, silu=1, batch=B, dim=D, seqlen=L,
                       x=x.data_ptr(), weight=w.data_ptr(), weight_c_stride=W, weight_width_stride=1,
                       bias=b.data_ptr(), dout=dout.data_ptr(), dx=dx.data_ptr(),
                       dweight=dw.data_ptr(), dweight_c_stride=W, dweight_width_stride=1, dbias=db.data_ptr(),
                       accumulate=0)
    for name, t in (("x", x), ("dout", dout), ("dx", dx)):
        for k, v in s(t).items():
            setattr(p, f"{name}_{k}_stride", v)
    return p


def _inputs(seed, itype, channel_last, B=3, D=72, L=333, W=4):
    torch.manual_seed(seed)
    mk = (lambda: torch.randn(B, L, D, device="cuda", dtype=itype).transpose(1, 2)) if channel_last else \
         (lambda: torch.randn(B, D, L, device="cuda", dtype=itype))
    x, dout = mk(), mk()
    w = torch.randn(D, W, device="cuda")
    b = torch.randn(D, device="cuda")
    return x, w, b, dout


@pytest.mark.parametrize("channel_last", [False, True])
@pytest.mark.parametrize("itype", [torch.float32, torch.bfloat16])
def test_noalloc_matches_workspace_entry_point(itype, channel_last):
    lib = cabi.load()
    for call, seed in enumerate((11, 12)):          # two calls in a row on the shared scratch
        x, w, b, dout = _inputs(seed, itype, channel_last)
        ref = [torch.empty_like(x), torch.empty(w.shape, device="cuda"), torch.empty(b.shape, device="cuda")]
        got = [torch.empty_like(x), torch.empty(w.shape, device="cuda"), torch.empty(b.shape, device="cuda")]
        # existing entry point: caller workspace
        p = _params(x, w, b, dout, *ref, channel_last)
        n = lib.cc1d_bwd_workspace_bytes(ctypes.byref(p))
        assert 0 < n <= SCRATCH_BYTES
        ws = torch.empty(n, dtype=torch.uint8, device="cuda")
        p.workspace, p.workspace_bytes = ws.data_ptr(), n
        assert lib.cc1d_bwd(ctypes.byref(p), _stream()) == 0
        # new entry point: no workspace handed over at all
        q = _params(x, w, b, dout, *got, channel_last)
        q.workspace, q.workspace_bytes = None, 0
        torch.cuda.synchronize()
        free_before, torch_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        assert lib.cc1d_bwd_noalloc(ctypes.byref(q), _stream()) == 0, f"call {call}"
        torch.cuda.synchronize()
        if call == 1:
            # the stated property: nothing was allocated on the device, by the driver or by torch
            # (checked on the second call: the very first call on a device may load the library's
            # device code, which the driver accounts for)
            # (device allocations come in chunks of at least 2 MiB: anything less is not one)
            assert free_before - torch.cuda.mem_get_info()[0] < (1 << 20)
            assert torch.cuda.memory_allocated() == torch_before
        assert_close(got[0], ref[0], TOL[itype], f"dx (call {call})")
        assert_close_sum(got[1], ref[1], 2e-5, f"dweight (call {call})")
        assert_close_sum(got[2], ref[2], 2e-5, f"dbias (call {call})")
        # same kernels, same fixed summation order: the bits agree as well
        assert all(torch.equal(a, c) for a, c in zip(got, ref))


def _fake_channel_first(batch, dim, seqlen, fake):
    return cabi.BwdParams(itype=cabi.BF16, wtype=cabi.F32, width=4, silu=1, batch=batch, dim=dim, seqlen=seqlen,
                          x=fake, x_batch_stride=dim * seqlen, x_c_stride=seqlen, x_l_stride=1,
                          weight=0x1000, weight_c_stride=4, weight_width_stride=1,
                          dout=fake, dout_batch_stride=dim * seqlen, dout_c_stride=seqlen, dout_l_stride=1,
                          dx=fake, dx_batch_stride=dim * seqlen, dx_c_stride=seqlen, dx_l_stride=1,
                          dweight=0x1000, dweight_c_stride=4, dweight_width_stride=1)


def test_noalloc_rejects_problems_beyond_its_scratch():
    lib = cabi.load()
    # (32, 8192, 8192) bf16 channel-first, rows NOT 16-byte aligned (pointers at 0x1002): the
    # element-wise tiling leaves one partial row per 256 elements = 32 * 8192 * 32 * 5 * 4 B = 168 MB,
    # more than the built-in 8 MiB.  The size test comes before any launch, so the pointers are
    # never dereferenced.
    p = _fake_channel_first(32, 8192, 8192, 0x1002)
    assert lib.cc1d_bwd_workspace_bytes(ctypes.byref(p)) > SCRATCH_BYTES
    rc = lib.cc1d_bwd_noalloc(ctypes.byref(p), _stream())
    assert rc == 15
    assert b"cc1d_bwd_noalloc" in lib.cc1d_status_str(rc)


def test_noalloc_limit_follows_the_tiling_that_runs():
    """cc1d_bwd_workspace_bytes() answers for the worse of the two channel-first tilings because it
    may be asked before the tensors exist.  cc1d_bwd_noalloc knows the pointers: an aligned
    problem whose vector tiling fits the built-in scratch is served even where the conservative
    figure exceeds it."""
    lib = cabi.load()
    B, D, L, W = 4, 4096, 8192, 4          # conservative: 4*4096*32*5*4 B = 10.5 MB; vector tiling: far less
    torch.manual_seed(13)
    x = torch.randn(B, D, L, device="cuda", dtype=torch.bfloat16)
    dout = torch.randn_like(x)
    w, b = torch.randn(D, W, device="cuda"), torch.randn(D, device="cuda")
    ref = [torch.empty_like(x), torch.empty_like(w), torch.empty_like(b)]
    got = [torch.empty_like(x), torch.empty_like(w), torch.empty_like(b)]
    p = _params(x, w, b, dout, *ref, False)
    n = lib.cc1d_bwd_workspace_bytes(ctypes.byref(p))
    assert n > SCRATCH_BYTES
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ws.data_ptr(), n
    assert lib.cc1d_bwd(ctypes.byref(p), _stream()) == 0
    q = _params(x, w, b, dout, *got, False)
    assert lib.cc1d_bwd_noalloc(ctypes.byref(q), _stream()) == 0
    torch.cuda.synchronize()
    assert all(torch.equal(a, c) for a, c in zip(got, ref))


def test_noalloc_on_a_second_device():
    """The scratch address is looked up per device; the entry point works on every GPU of the process."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    lib = cabi.load()
    with torch.cuda.device(1):
        torch.manual_seed(14)
        x = torch.randn(2, 64, 512, device="cuda:1", dtype=torch.bfloat16)
        dout = torch.randn_like(x)
        w, b = torch.randn(64, 4, device="cuda:1"), torch.randn(64, device="cuda:1")
        ref = [torch.empty_like(x), torch.empty_like(w), torch.empty_like(b)]
        got = [torch.empty_like(x), torch.empty_like(w), torch.empty_like(b)]
        p = _params(x, w, b, dout, *ref, False)
        n = lib.cc1d_bwd_workspace_bytes(ctypes.byref(p))
        ws = torch.empty(n, dtype=torch.uint8, device="cuda:1")
        p.workspace, p.workspace_bytes = ws.data_ptr(), n
        s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert lib.cc1d_bwd(ctypes.byref(p), s) == 0
        q = _params(x, w, b, dout, *got, False)
        assert lib.cc1d_bwd_noalloc(ctypes.byref(q), s) == 0
        torch.cuda.synchronize()
        assert all(torch.equal(a, c) for a, c in zip(got, ref))
