"""The float64 PyTorch statement used for large GPU checks, against the CPU oracle (no GPU)."""
import pytest
import torch

import oracle
from conftest import assert_close
from torch_ref import conv_grads64


@pytest.mark.parametrize("width", [2, 3, 4])
@pytest.mark.parametrize("mode", ["plain", "states", "seq_idx"])
@pytest.mark.parametrize("silu", [False, True])
def test_torch_ref_matches_oracle(width, mode, silu):
    torch.manual_seed(width * 7 + silu)
    B, D, L = 2, 5, 23
    x, w, b, dout = torch.randn(B, D, L), torch.randn(D, width), torch.randn(D), torch.randn(B, D, L)
    act = "silu" if silu else None
    sidx = ini = dfin = None
    if mode == "states":
        ini, dfin = torch.randn(B, D, width - 1), torch.randn(B, D, width - 1)
    if mode == "seq_idx":
        sidx = torch.tensor([[0] * 5 + [1] * 1 + [2] * 12 + [-1] * 5, [3] * 23], dtype=torch.int32)
    r = conv_grads64(x, w, b, dout, sidx, ini, dfin, act)
    o = oracle.fwd(x, w, b, seq_idx=sidx, initial_states=ini, return_final_states=mode == "states", activation=act)
    if mode == "states":
        o, fs = o
        assert torch.equal(fs, r["final_states"])
    assert_close(r["out"], o, 1e-12, "out")
    g = oracle.bwd(x, w, b, dout, seq_idx=sidx, initial_states=ini, dfinal_states=dfin, activation=act)
    for k in ("dx", "dweight", "dbias", "dinitial_states"):
        if g[k] is not None:
            assert_close(r[k], g[k], 1e-11, k)
