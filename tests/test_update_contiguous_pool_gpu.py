"""Decode update with a contiguous (entries, dim, state_len) pool and x / out stored
(batch, dim, seqlen) contiguous: 1 to 4 tokens per step, linear (state_len == width-1 or width)
and the circular buffer of 8 slots, with gathered and padded batch entries.  Against the CPU
oracle; the pool must come out bit-exact."""
import pytest
import torch

import oracle
from conftest import TOL, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("itype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("width", [2, 3, 4])
@pytest.mark.parametrize("seqlen", [1, 2, 3, 4])
@pytest.mark.parametrize("mode", ["linear_w-1", "linear_w", "circular8"])
def test_update_contiguous_pool(mode, seqlen, width, itype):
    from causal_conv1d_b200 import causal_conv1d_update
    torch.manual_seed(seqlen * 10 + width)
    batch, entries, dim = 24, 60, 264
    S = {"linear_w-1": width - 1, "linear_w": width, "circular8": 8}[mode]
    x = torch.randn(batch, dim, seqlen, device=DEV, dtype=itype)
    pool = torch.randn(entries, dim, S, device=DEV, dtype=itype)
    w = torch.randn(dim, width, device=DEV)
    b = torch.randn(dim, device=DEV)
    idx = torch.randperm(entries)[:batch].int()
    idx[3] = idx[17] = -1                                   # padded entries
    idx = idx.to(DEV)
    cache = torch.randint(0, 10000, (batch,), dtype=torch.int32, device=DEV) if mode == "circular8" else None
    before = pool.clone()
    o_out, o_pool = oracle.update(x, pool, w, b, activation="silu", cache_seqlens=cache, conv_state_indices=idx)
    out = causal_conv1d_update(x, pool, w, b, activation="silu", cache_seqlens=cache, conv_state_indices=idx)
    assert torch.equal(pool.cpu(), o_pool.to(itype)), "pool must be bit-exact"
    assert torch.all(out[idx < 0] == 0)
    assert_close(out, o_out.to(itype), TOL[itype], "out")
    touched = torch.zeros(entries, dtype=torch.bool, device=DEV)
    touched[idx[idx >= 0].long()] = True
    assert torch.equal(pool[~touched], before[~touched])
    # the same step with x / out token-major (another kernel) gives the same bits
    pool2 = before.clone()
    out2 = causal_conv1d_update(x.transpose(1, 2).contiguous().transpose(1, 2), pool2, w, b, activation="silu",
                                cache_seqlens=cache, conv_state_indices=idx)
    assert torch.equal(pool2, pool)
    assert_close(out2, out, TOL[itype], "out, other kernel")
