"""Public API: ``causal_conv1d_fn``, ``CausalConv1dFn`` and ``causal_conv1d_update`` with
the signatures, argument normalisation and error behaviour of the reference
(``causal_conv1d/causal_conv1d_interface.py:9-129,174-202``).  ``causal_conv1d_ref`` and
``causal_conv1d_update_ref`` (``:132-171,205-242``), the PyTorch statements callers compare
against, are re-exported from ``torch_reference``; the CUDA entry points never call them."""
import torch

from causal_conv1d_b200.cpp_functions import (
    causal_conv1d_bwd_function,
    causal_conv1d_fwd_function,
    causal_conv1d_update_function,
)
from causal_conv1d_b200.torch_reference import causal_conv1d_ref, causal_conv1d_update_ref  # noqa: F401

_ACTIVATIONS = (None, "silu", "swish")


def _unit_inner_stride(t: torch.Tensor) -> bool:
    return t.stride(2) == 1 or t.stride(1) == 1


class CausalConv1dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias=None, seq_idx=None, initial_states=None, return_final_states=False,
                final_states_out=None, activation=None):
        if activation not in _ACTIVATIONS:
            raise NotImplementedError("activation must be None, silu, or swish")
        if not _unit_inner_stride(x):
            x = x.contiguous()
        if bias is not None:
            bias = bias.contiguous()
        if seq_idx is not None:
            assert initial_states is None, "initial_states must be None if seq_idx is not None"
            assert not return_final_states, "If seq_idx is not None, we don't return final_states_out"
            seq_idx = seq_idx.contiguous()
        if initial_states is not None and not _unit_inner_stride(initial_states):
            initial_states = initial_states.contiguous()
        if return_final_states:
            assert x.stride(1) == 1, "Only channel-last layout support returning final_states_out"
            if final_states_out is not None:
                assert _unit_inner_stride(final_states_out)
            else:
                batch, dim, _ = x.shape
                width = weight.shape[1]
                final_states_out = torch.empty(batch, width - 1, dim, device=x.device, dtype=x.dtype).transpose(1, 2)
        else:
            final_states_out = None
        ctx.activation = activation in ("silu", "swish")
        out = causal_conv1d_fwd_function(x, weight, bias, seq_idx, initial_states, final_states_out, ctx.activation)
        ctx.save_for_backward(x, weight, bias, seq_idx, initial_states)
        ctx.return_final_states = return_final_states
        ctx.return_dinitial_states = initial_states is not None and initial_states.requires_grad
        if return_final_states:
            return out, final_states_out
        return out

    @staticmethod
    def backward(ctx, dout, *args):
        x, weight, bias, seq_idx, initial_states = ctx.saved_tensors
        dfinal_states = args[0] if ctx.return_final_states else None
        if not _unit_inner_stride(dout):
            dout = dout.contiguous()
        dx, dweight, dbias, dinitial_states = causal_conv1d_bwd_function(
            x, weight, bias, dout, seq_idx, initial_states, dfinal_states, None,
            ctx.return_dinitial_states, ctx.activation,
        )
        return (
            dx,
            dweight,
            dbias if bias is not None else None,
            None,
            dinitial_states if initial_states is not None else None,
            None,
            None,
            None,
        )


def causal_conv1d_fn(x, weight, bias=None, seq_idx=None, initial_states=None, return_final_states=False,
                     final_states_out=None, activation=None):
    """
    x: (batch, dim, seqlen)
    weight: (dim, width)
    bias: (dim,)
    seq_idx: (batch, seqlen)
    initial_states: (batch, dim, width - 1)
    final_states_out: (batch, dim, width - 1), to be written to
    activation: either None or "silu" or "swish"

    out: (batch, dim, seqlen)
    """
    return CausalConv1dFn.apply(x, weight, bias, seq_idx, initial_states, return_final_states,
                                final_states_out, activation)


def causal_conv1d_update(x, conv_state, weight, bias=None, activation=None, cache_seqlens=None,
                         conv_state_indices=None):
    """
    x: (batch, dim) or (batch, dim, seqlen)
    conv_state: (batch, dim, state_len), where state_len >= width - 1; updated in place
    weight: (dim, width)
    bias: (dim,)
    cache_seqlens: (batch,), dtype int32.
        If not None, conv_state is a circular buffer: x is written starting at index
        cache_seqlens % state_len.
    conv_state_indices: (batch,), dtype int32.
        If not None, conv_state is a pool (entries, dim, state_len) and entry
        conv_state_indices[b] is the state of batch row b; a negative index marks a padded
        row (zero output, no state touched).

    out: (batch, dim) or (batch, dim, seqlen)
    """
    if activation not in _ACTIVATIONS:
        raise NotImplementedError("activation must be None, silu, or swish")
    silu = activation in ("silu", "swish")
    squeeze = x.dim() == 2
    if squeeze:
        x = x.unsqueeze(-1)
    out = causal_conv1d_update_function(x, conv_state, weight, bias, silu, cache_seqlens, conv_state_indices)
    return out.squeeze(-1) if squeeze else out
