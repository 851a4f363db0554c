"""The C-ABI shared library without a GPU: it loads, exports every symbol the header
declares, and rejects bad parameter blocks with the documented status before touching CUDA."""
import ctypes

import pytest

import cabi

FAKE = 0x1000  # never dereferenced: validation fails first


@pytest.fixture(scope="module")
def lib():
    import causal_conv1d_b200._build as b
    b.build_kernels()
    return cabi.load()


def test_exports_every_declared_symbol(lib):
    names = cabi.declared_symbols()
    assert {"cc1d_fwd", "cc1d_bwd", "cc1d_bwd_workspace_bytes", "cc1d_update", "cc1d_varlen_states",
            "cc1d_status_str", "cc1d_abi_version"} <= set(names)
    for n in names:
        assert hasattr(lib, n), f"libcc1d.so does not export {n}"
    assert lib.cc1d_abi_version() >= 4


def test_struct_sizes_match_header():
    # all fields are 4- or 8-byte scalars laid out without surprises; spot-check total sizes
    assert ctypes.sizeof(cabi.FwdParams) == 16 + 3 * 8 + 8 + 24 + 8 + 16 + 8 + 8 + 24 + 8 + 8 + 24 + 8 + 24
    assert ctypes.sizeof(cabi.VarlenParams) == 8 + 4 * 8 + 8 + 16 + 8 + 8 + 24


def _fwd(**kw):
    p = cabi.FwdParams(itype=cabi.BF16, wtype=cabi.BF16, width=4, silu=1, batch=2, dim=64, seqlen=128,
                       x=FAKE, x_batch_stride=64 * 128, x_c_stride=128, x_l_stride=1,
                       weight=FAKE, weight_c_stride=4, weight_width_stride=1,
                       out=FAKE, out_batch_stride=64 * 128, out_c_stride=128, out_l_stride=1)
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("kw,code,text", [
    (dict(width=5), 3, "width between 2 and 4"),
    (dict(width=1), 3, "width between 2 and 4"),
    (dict(itype=7), 2, "dtype"),
    (dict(x=0), 1, "NULL"),
    (dict(out=0), 1, "NULL"),
    (dict(batch=-1), 4, "sizes"),
    (dict(x_c_stride=3, x_l_stride=2), 5, "contiguous"),
    (dict(dim=60, x_c_stride=1, x_l_stride=64), 6, "divisible by 8"),
    (dict(x_c_stride=1, x_l_stride=68), 7, "multiples of 8"),
    (dict(seq_idx=FAKE), 8, "channel last"),
    (dict(x=FAKE + 1), 12, "aligned"),
    # seq_idx excludes states (channel-last block: dim 64, tokens 128 apart by 64 elements)
    (dict(x_c_stride=1, x_l_stride=64, out_c_stride=1, out_l_stride=64, seq_idx=FAKE, initial_states=FAKE,
          initial_states_c_stride=1), 18, "seq_idx cannot be combined"),
    (dict(x_c_stride=1, x_l_stride=64, out_c_stride=1, out_l_stride=64, seq_idx=FAKE, final_states=FAKE,
          final_states_c_stride=1), 18, "seq_idx cannot be combined"),
    # token positions are 32-bit in the channel-last kernels
    (dict(batch=1, seqlen=(1 << 31) - 8, x_c_stride=1, x_l_stride=64, out_c_stride=1, out_l_stride=64), 13, "index range"),
])
def test_fwd_rejects(lib, kw, code, text):
    p = _fwd(**kw)
    rc = lib.cc1d_fwd(ctypes.byref(p), None)
    assert rc == code
    assert text in lib.cc1d_status_str(rc).decode()


def test_update_rejects(lib):
    p = cabi.UpdateParams(itype=cabi.F32, wtype=cabi.F32, width=4, silu=0, batch=2, dim=8, seqlen=1,
                          x=FAKE, weight=FAKE, out=FAKE, conv_state=FAKE, conv_state_len=2)
    assert lib.cc1d_update(ctypes.byref(p), None) == 10   # state_len < width - 1
    p.conv_state_len = 3
    p.conv_state = 0
    assert lib.cc1d_update(ctypes.byref(p), None) == 1
    assert lib.cc1d_update(None, None) == 1


def test_bwd_workspace_and_rejects(lib):
    p = cabi.BwdParams(itype=cabi.BF16, wtype=cabi.F32, width=4, silu=1, batch=8, dim=5120, seqlen=2048,
                       x=FAKE, x_batch_stride=5120 * 2048, x_c_stride=2048, x_l_stride=1,
                       weight=FAKE, weight_c_stride=4, weight_width_stride=1,
                       dout=FAKE, dout_batch_stride=5120 * 2048, dout_c_stride=2048, dout_l_stride=1,
                       dx=FAKE, dx_batch_stride=5120 * 2048, dx_c_stride=2048, dx_l_stride=1,
                       dweight=FAKE, dweight_c_stride=4, dweight_width_stride=1)
    n = lib.cc1d_bwd_workspace_bytes(ctypes.byref(p))
    # one fp32 row of width+1 per (batch, channel, 256-element tile): 8 * 5120 * 8 * 5 * 4 bytes
    assert n == 8 * 5120 * 8 * 5 * 4
    assert lib.cc1d_bwd(ctypes.byref(p), None) == 11          # workspace missing
    p.workspace, p.workspace_bytes = FAKE, n - 1
    assert lib.cc1d_bwd(ctypes.byref(p), None) == 11          # workspace too small
    p.bias = FAKE                                             # bias without dbias
    assert lib.cc1d_bwd(ctypes.byref(p), None) == 1
    p.width = 9
    assert lib.cc1d_bwd_workspace_bytes(ctypes.byref(p)) == 0
    # channel-last problem: partial rows per (batch, group of 4 chunks); 16-bit I/O picks the chunk
    # length by the waves of CTAs it makes (here 160 tokens: 52 groups), fp32 keeps 128 tokens
    q = cabi.BwdParams(itype=cabi.BF16, wtype=cabi.BF16, width=4, silu=1, batch=1, dim=5376, seqlen=32768,
                       x=FAKE, x_batch_stride=5376 * 32768, x_c_stride=1, x_l_stride=5376)
    assert lib.cc1d_bwd_workspace_bytes(ctypes.byref(q)) == 52 * 5376 * 5 * 4
    q.itype = cabi.F32
    assert lib.cc1d_bwd_workspace_bytes(ctypes.byref(q)) == 64 * 5376 * 5 * 4
    # (8,5120,2048) channel-last: 128-token chunks make fewer waves than 160 here (4 groups per batch row)
    r = cabi.BwdParams(itype=cabi.BF16, wtype=cabi.BF16, width=4, silu=1, batch=8, dim=5120, seqlen=2048,
                       x=FAKE, x_batch_stride=5120 * 2048, x_c_stride=1, x_l_stride=5120)
    assert lib.cc1d_bwd_workspace_bytes(ctypes.byref(r)) == 8 * 4 * 5120 * 5 * 4


def test_bwd_rejects_seq_idx_with_states_phase_and_long_sequences(lib):
    def block(**kw):
        p = cabi.BwdParams(itype=cabi.F32, wtype=cabi.F32, width=4, silu=1, batch=1, dim=64, seqlen=128,
                           x=FAKE, x_c_stride=1, x_l_stride=64, weight=FAKE, weight_c_stride=4, weight_width_stride=1,
                           dout=FAKE, dout_c_stride=1, dout_l_stride=64, dx=FAKE, dx_c_stride=1, dx_l_stride=64,
                           dweight=FAKE, dweight_c_stride=4, dweight_width_stride=1,
                           workspace=FAKE, workspace_bytes=1 << 40)
        for k, v in kw.items():
            setattr(p, k, v)
        return p
    for kw in (dict(initial_states=FAKE, initial_states_c_stride=1), dict(dfinal_states=FAKE),
               dict(dinitial_states=FAKE, dinitial_states_c_stride=1)):
        rc = lib.cc1d_bwd(ctypes.byref(block(seq_idx=FAKE, **kw)), None)
        assert rc == 18 and b"seq_idx cannot be combined" in lib.cc1d_status_str(rc)
    assert lib.cc1d_bwd(ctypes.byref(block(phase=3)), None) == 19
    # a channel-first dout beside a channel-last x: 16-bit types with 16-byte aligned rows only
    assert lib.cc1d_bwd(ctypes.byref(block(dout_c_stride=128, dout_l_stride=1)), None) == 5          # fp32
    assert lib.cc1d_bwd(ctypes.byref(block(itype=cabi.BF16, dout_c_stride=130, dout_l_stride=1)), None) == 5
    assert lib.cc1d_bwd(ctypes.byref(block(seqlen=(1 << 31) - 8)), None) == 13       # fp32: the non-TMA kernel
    p = _prefill(total_tokens=(1 << 31) - 8)
    assert lib.cc1d_prefill_varlen(ctypes.byref(p), None) == 13


def test_varlen_rejects(lib):
    p = cabi.VarlenParams(itype=9, total_tokens=4, dim=8, batch=1, state_len=2, x=FAKE, cu_seqlens=FAKE, states=FAKE)
    assert lib.cc1d_varlen_states(ctypes.byref(p), None) == 2
    p.itype, p.states = cabi.F16, 0
    assert lib.cc1d_varlen_states(ctypes.byref(p), None) == 1


def test_status_strings(lib):
    assert lib.cc1d_status_str(0) == b"ok"
    assert b"unknown" in lib.cc1d_status_str(999)


def _prefill(**kw):
    p = cabi.PrefillParams(itype=cabi.BF16, wtype=cabi.F32, width=4, silu=1, total_tokens=64, dim=64, nseq=2, state_len=3,
                           x=FAKE, x_l_stride=64, weight=FAKE, weight_c_stride=4, weight_width_stride=1,
                           out=FAKE, out_l_stride=64, seq_idx=FAKE, cu_seqlens=FAKE,
                           initial_states=FAKE, initial_states_batch_stride=192, initial_states_l_stride=64,
                           final_states=FAKE, final_states_batch_stride=192, final_states_l_stride=64)
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("kw,code", [
    (dict(width=1), 3),
    (dict(itype=9), 2),
    (dict(dim=60), 6),                       # channel-last rule: dim % 8 == 0
    (dict(state_len=2), 10),                 # shorter than width - 1
    (dict(nseq=-1), 4),
    (dict(cu_seqlens=0), 1),
    (dict(seq_idx=0), 1),
    (dict(x_l_stride=1), 5),
    (dict(final_states_l_stride=63), 12),    # state vectors are moved 16 bytes at a time
    (dict(initial_states=FAKE + 2), 12),
])
def test_prefill_varlen_rejects(lib, kw, code):
    p = _prefill(**kw)
    assert lib.cc1d_prefill_varlen(ctypes.byref(p), None) == code


def test_prefill_varlen_empty_problems_are_ok(lib):
    assert lib.cc1d_prefill_varlen(ctypes.byref(_prefill(dim=0)), None) == 0
    assert lib.cc1d_seq_idx_from_cu_seqlens(None, 0, 0, None, None) == 0
    assert lib.cc1d_seq_idx_from_cu_seqlens(None, 3, 10, None, None) == 1
    assert lib.cc1d_seq_idx_from_cu_seqlens(None, -1, 10, None, None) == 4


def test_struct_size_of_prefill_block():
    assert ctypes.sizeof(cabi.PrefillParams) == 16 + 4 * 8 + 2 * 8 + 4 * 8 + 2 * 8 + 4 * 8 + 3 * 8 + 3 * 8
