"""PyTorch statements of the three ops, under the names the reference exports for them:
``causal_conv1d_ref`` and ``causal_conv1d_update_ref``
(``causal_conv1d/causal_conv1d_interface.py:132-171,205-242``) and
``causal_conv1d_varlen_states_ref`` (``causal_conv1d/causal_conv1d_varlen.py:67-86``).

Callers of the reference (its own test file first of all) import these next to the CUDA
entry points and compare the two, so a drop-in has to carry them.  They are specifications
written with stock PyTorch operators, they run wherever their inputs live, and NOTHING in the
CUDA path of this package calls them: ``causal_conv1d_fn`` / ``causal_conv1d_update`` /
``causal_conv1d_varlen_states`` never fall back to them.

Arithmetic follows the reference's statement: the convolution runs in the dtype of ``weight``
and the result is cast back to the dtype of ``x`` after the activation.
"""
import torch
import torch.nn.functional as F

_ACTIVATIONS = (None, "silu", "swish")


def _depthwise_valid(xp, weight, bias):
    """out[b, c, t] = bias[c] + sum_k weight[c, k] * xp[b, c, t + k] (no padding)."""
    dim = weight.shape[0]
    return F.conv1d(xp, weight[:, None, :], bias, groups=dim)


def causal_conv1d_ref(x, weight, bias=None, initial_states=None, return_final_states=False,
                      final_states_out=None, activation=None):
    """
    x: (batch, dim, seqlen)
    weight: (dim, width)
    bias: (dim,)
    initial_states: (batch, dim, width - 1), the left context (zeros when None)
    final_states_out: (batch, dim, width - 1), written when given

    out: (batch, dim, seqlen), or (out, final_states) with return_final_states
    """
    if activation not in _ACTIVATIONS:
        raise NotImplementedError("activation must be None, silu, or swish")
    io_dtype = x.dtype
    batch, dim, seqlen = x.shape
    width = weight.shape[1]
    xw = x.to(weight.dtype)
    if initial_states is None:
        head = xw.new_zeros(batch, dim, width - 1)
    else:
        head = initial_states
    xp = torch.cat([head, xw], dim=-1)                 # (batch, dim, width - 1 + seqlen)
    y = _depthwise_valid(xp, weight, bias)             # (batch, dim, seqlen)
    if activation is not None:
        y = F.silu(y)
    out = y.to(io_dtype)
    if not return_final_states:
        return out
    final_states = xp[..., seqlen:].to(io_dtype)       # the last width - 1 entries of [head | x]
    if final_states_out is not None:
        final_states_out.copy_(final_states)
        final_states = final_states_out
    return out, final_states


def causal_conv1d_update_ref(x, conv_state, weight, bias=None, activation=None, cache_seqlens=None):
    """
    x: (batch, dim) or (batch, dim, seqlen)
    conv_state: (batch, dim, state_len), state_len >= width - 1; updated in place
    weight: (dim, width)
    bias: (dim,)
    cache_seqlens: (batch,) int32 or None.  When given, conv_state is a circular buffer: the
        window is the width - 1 entries before position cache_seqlens % state_len, and x is
        written starting at that position (both wrap around).

    out: (batch, dim) or (batch, dim, seqlen)
    """
    if activation not in _ACTIVATIONS:
        raise NotImplementedError("activation must be None, silu, or swish")
    io_dtype = x.dtype
    squeeze = x.dim() == 2
    if squeeze:
        x = x[..., None]
    batch, dim, seqlen = x.shape
    width = weight.shape[1]
    state_len = conv_state.shape[-1]
    assert conv_state.shape == (batch, dim, state_len)
    assert weight.shape == (dim, width)
    if cache_seqlens is None:
        joined = torch.cat([conv_state, x], dim=-1)
        window = joined.to(weight.dtype)
        conv_state.copy_(joined[..., seqlen:])          # the newest state_len entries
    else:
        start = cache_seqlens.long()[:, None]            # (batch, 1)
        back = torch.arange(-(width - 1), 0, device=x.device)[None, :]
        ahead = torch.arange(seqlen, device=x.device)[None, :]
        read_at = torch.remainder(start + back, state_len)[:, None, :].expand(batch, dim, width - 1)
        write_at = torch.remainder(start + ahead, state_len)[:, None, :].expand(batch, dim, seqlen)
        window = torch.cat([torch.gather(conv_state, 2, read_at), x], dim=-1).to(weight.dtype)
        conv_state.scatter_(2, write_at, x)
    y = _depthwise_valid(window, weight, bias)[..., -seqlen:]
    if activation is not None:
        y = F.silu(y)
    if squeeze:
        y = y[..., 0]
    return y.to(io_dtype)


def causal_conv1d_varlen_states_ref(x, cu_seqlens, state_len):
    """
    x: (total_tokens, dim); cu_seqlens: (batch + 1,), sorted, from 0.
    states[b, :, state_len - n:] = x[end_b - n : end_b].T with n = min(state_len, len_b);
    the slots before that are zero.  Forward only.

    states: (batch, dim, state_len), stored channel-last (stride(1) == 1)
    """
    dim = x.shape[1]
    bounds = [int(v) for v in cu_seqlens.tolist()]
    batch = len(bounds) - 1
    states = torch.zeros(batch, state_len, dim, dtype=x.dtype, device=x.device).transpose(1, 2)
    for b in range(batch):
        end = bounds[b + 1]
        n = min(state_len, end - bounds[b])
        if n > 0:
            states[b, :, state_len - n:] = x[end - n:end].transpose(0, 1)
    return states
