"""TEST INFRASTRUCTURE — ctypes front end of the CPU oracle (see ``cc1d_oracle.c``).

The C functions restate the reference's PyTorch oracle functions
(``causal_conv1d_ref`` causal_conv1d/causal_conv1d_interface.py:132-171,
``causal_conv1d_update_ref`` :205-242, ``causal_conv1d_varlen_states_ref``
causal_conv1d/causal_conv1d_varlen.py:67-86) and the gradient autograd derives for the
first.  They are pinned against outputs of those functions stored under
``tests/golden/``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import time

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcc1d_oracle.so")
_lib = None

_i64 = ctypes.c_int64
_int = ctypes.c_int
_ptr = ctypes.c_void_p


def build(force: bool = False) -> str:
    """Compile the C oracle with gcc (``make -C oracle``); returns the library path."""
    src = [os.path.join(_HERE, f) for f in ("cc1d_oracle.c", "cc1d_oracle_impl.inc", "Makefile")]
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libcc1d_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        for suf in ("_f64", "_f32"):
            getattr(_lib, "cc1d_oracle_fwd" + suf).argtypes = [_i64, _i64, _i64, _int, _int] + [_ptr] * 7
            getattr(_lib, "cc1d_oracle_bwd" + suf).argtypes = [_i64, _i64, _i64, _int, _int] + [_ptr] * 11
            getattr(_lib, "cc1d_oracle_update" + suf).argtypes = [_i64, _i64, _i64, _int, _int, _i64] + [_ptr] * 7
            getattr(_lib, "cc1d_oracle_varlen_states" + suf).argtypes = [_i64, _i64, _i64] + [_ptr] * 3
            for n in ("fwd", "bwd", "update", "varlen_states"):
                getattr(_lib, f"cc1d_oracle_{n}{suf}").restype = None
        _lib.cc1d_oracle_max_threads.restype = _int
        _lib.cc1d_oracle_set_threads.argtypes = [_int]
    return _lib


def max_threads() -> int:
    return int(lib().cc1d_oracle_max_threads())


def set_threads(n: int) -> None:
    lib().cc1d_oracle_set_threads(int(n))


def round_to(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round a float64 oracle result to an I/O dtype (one rounding, like the kernels)."""
    return t.to(dtype)


def _dense(t, np_dtype):
    """torch tensor (any dtype/layout/device) -> C-contiguous numpy array, or None."""
    if t is None:
        return None
    tt = t.detach().cpu()
    if tt.is_floating_point():
        tt = tt.to(torch.float64 if np_dtype == np.float64 else torch.float32)
    return np.ascontiguousarray(tt.contiguous().numpy().astype(np_dtype, copy=False))


def _p(a):
    return None if a is None else a.ctypes.data_as(_ptr)


def fwd(x, weight, bias=None, seq_idx=None, initial_states=None, return_final_states=False,
        activation=None):
    """float64 forward.  Returns out (batch, dim, seqlen) [, final_states (batch, dim, width-1)]."""
    assert activation in (None, "silu", "swish")
    batch, dim, seqlen = x.shape
    width = weight.shape[1]
    xa, wa, ba = _dense(x, np.float64), _dense(weight, np.float64), _dense(bias, np.float64)
    sa, ia = _dense(seq_idx, np.int32), _dense(initial_states, np.float64)
    out = np.empty((batch, dim, seqlen), np.float64)
    fs = np.empty((batch, dim, width - 1), np.float64) if return_final_states else None
    lib().cc1d_oracle_fwd_f64(batch, dim, seqlen, width, int(activation is not None),
                              _p(xa), _p(wa), _p(ba), _p(sa), _p(ia), _p(out), _p(fs))
    out_t = torch.from_numpy(out)
    return (out_t, torch.from_numpy(fs)) if return_final_states else out_t


def bwd(x, weight, bias, dout, seq_idx=None, initial_states=None, dfinal_states=None,
        activation=None):
    """float64 backward.  Returns dict(dx, dweight, dbias|None, dinitial_states|None)."""
    assert activation in (None, "silu", "swish")
    batch, dim, seqlen = x.shape
    width = weight.shape[1]
    xa, wa, ba = _dense(x, np.float64), _dense(weight, np.float64), _dense(bias, np.float64)
    da = _dense(dout, np.float64)
    sa, ia = _dense(seq_idx, np.int32), _dense(initial_states, np.float64)
    dfa = _dense(dfinal_states, np.float64)
    dx = np.empty((batch, dim, seqlen), np.float64)
    dw = np.empty((dim, width), np.float64)
    db = np.empty((dim,), np.float64) if bias is not None else None
    dini = np.empty((batch, dim, width - 1), np.float64) if initial_states is not None else None
    lib().cc1d_oracle_bwd_f64(batch, dim, seqlen, width, int(activation is not None),
                              _p(xa), _p(wa), _p(ba), _p(da), _p(sa), _p(ia), _p(dfa),
                              _p(dx), _p(dw), _p(db), _p(dini))
    return {
        "dx": torch.from_numpy(dx),
        "dweight": torch.from_numpy(dw),
        "dbias": None if db is None else torch.from_numpy(db),
        "dinitial_states": None if dini is None else torch.from_numpy(dini),
    }


def update(x, conv_state, weight, bias=None, activation=None, cache_seqlens=None,
           conv_state_indices=None):
    """float64 decode update.  Returns (out, new_conv_state); the input state is NOT modified.

    x: (batch, dim) or (batch, dim, seqlen); conv_state: (entries, dim, state_len).
    State values are only copied, so rounding new_conv_state to the I/O dtype is exact.
    """
    assert activation in (None, "silu", "swish")
    squeeze = x.dim() == 2
    if squeeze:
        x = x.unsqueeze(-1)
    batch, dim, seqlen = x.shape
    width = weight.shape[1]
    state_len = conv_state.shape[-1]
    xa, wa, ba = _dense(x, np.float64), _dense(weight, np.float64), _dense(bias, np.float64)
    st = _dense(conv_state, np.float64).copy()
    ca, ia = _dense(cache_seqlens, np.int32), _dense(conv_state_indices, np.int32)
    out = np.empty((batch, dim, seqlen), np.float64)
    lib().cc1d_oracle_update_f64(batch, dim, seqlen, width, int(activation is not None), state_len,
                                 _p(xa), _p(st), _p(wa), _p(ba), _p(ca), _p(ia), _p(out))
    out_t = torch.from_numpy(out)
    if squeeze:
        out_t = out_t.squeeze(-1)
    return out_t, torch.from_numpy(st)


def varlen_states(x, cu_seqlens, state_len):
    """x: (total_tokens, dim) -> float64 states (batch, dim, state_len)."""
    total, dim = x.shape
    batch = cu_seqlens.shape[0] - 1
    xa = _dense(x, np.float64)
    cu = _dense(cu_seqlens, np.int64)
    states = np.empty((batch, dim, state_len), np.float64)
    lib().cc1d_oracle_varlen_states_f64(dim, batch, state_len, _p(xa), _p(cu), _p(states))
    return torch.from_numpy(states)


# ----------------------------------------------------------------------------------
# float32 variants, used only to TIME the CPU port (cpu_baseline in bench.py).
# Inputs must already be dense float32 / int32 numpy arrays; outputs are preallocated
# by the caller so that the timed region holds arithmetic only.
# ----------------------------------------------------------------------------------
def fwd_f32_timed(x, weight, bias, out, width, silu, repeats=1):
    batch, dim, seqlen = x.shape
    f = lib().cc1d_oracle_fwd_f32
    t0 = time.perf_counter()
    for _ in range(repeats):
        f(batch, dim, seqlen, width, int(silu), _p(x), _p(weight), _p(bias), None, None, _p(out), None)
    return (time.perf_counter() - t0) / repeats


def bwd_f32_timed(x, weight, bias, dout, dx, dweight, dbias, width, silu, repeats=1):
    batch, dim, seqlen = x.shape
    f = lib().cc1d_oracle_bwd_f32
    t0 = time.perf_counter()
    for _ in range(repeats):
        f(batch, dim, seqlen, width, int(silu), _p(x), _p(weight), _p(bias), _p(dout), None, None, None,
          _p(dx), _p(dweight), _p(dbias), None)
    return (time.perf_counter() - t0) / repeats


def update_f32_timed(x, conv_state, weight, bias, out, width, silu, repeats=1):
    batch, dim, seqlen = x.shape
    state_len = conv_state.shape[-1]
    f = lib().cc1d_oracle_update_f32
    t0 = time.perf_counter()
    for _ in range(repeats):
        f(batch, dim, seqlen, width, int(silu), state_len, _p(x), _p(conv_state), _p(weight), _p(bias),
          None, None, _p(out))
    return (time.perf_counter() - t0) / repeats


def prefill_varlen(x, weight, bias, cu_seqlens, conv_states=None, state_indices=None,
                   has_initial_state=None, activation=None):
    """float64 packed-varlen prefill with per-sequence states, composed from ``fwd`` (which
    restates causal_conv1d_ref, causal_conv1d/causal_conv1d_interface.py:132-171) one sequence
    at a time — the loop the reference's own seq_idx test runs
    (tests/test_causal_conv1d.py:448-454), here with ``initial_states``.

    x: (total_tokens, dim); conv_states: (rows, dim, state_len) or None.
    Returns (out (total_tokens, dim) float64, new_conv_states float64 or None); tokens at or
    after cu_seqlens[-1] output zero.  The final state of a sequence is the last state_len
    entries of [prefix | x_s] (for state_len == width-1 that is the reference's final_states,
    without a prefix it is causal_conv1d_varlen_states_ref, causal_conv1d_varlen.py:67-86).
    """
    total, dim = x.shape
    width = weight.shape[1]
    cu = [int(v) for v in cu_seqlens.detach().cpu().tolist()]
    xd = x.detach().cpu().to(torch.float64)
    out = torch.zeros(total, dim, dtype=torch.float64)
    new_states = None if conv_states is None else conv_states.detach().cpu().to(torch.float64).clone()
    S = None if conv_states is None else conv_states.shape[-1]
    for s in range(len(cu) - 1):
        beg, end = cu[s], cu[s + 1]
        row = s if state_indices is None else int(state_indices[s])
        prefixed = conv_states is not None and row >= 0 and (has_initial_state is None or bool(has_initial_state[s]))
        prefix = (conv_states[row].detach().cpu().to(torch.float64) if prefixed
                  else (torch.zeros(dim, S, dtype=torch.float64) if S is not None else None))
        xs = xd[beg:end].T.unsqueeze(0)   # (1, dim, len)
        if end > beg:
            ini = prefix[:, S - (width - 1):].unsqueeze(0) if prefixed else None
            out[beg:end] = fwd(xs, weight, bias, initial_states=ini, activation=activation)[0].T
        if new_states is not None and row >= 0:
            new_states[row] = torch.cat([prefix, xs[0]], dim=1)[:, -S:]
    return out, new_states
