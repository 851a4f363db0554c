"""``causal_conv1d_varlen_states`` — same signature as the reference's Triton-backed
function (``causal_conv1d/causal_conv1d_varlen.py:35-64``), served by a CUDA kernel.
``causal_conv1d_varlen_states_ref`` (``:67-86``) is re-exported from ``torch_reference``."""
from torch import Tensor

from causal_conv1d_b200.cpp_functions import (
    causal_conv1d_prefill_varlen_function,
    causal_conv1d_varlen_states_function,
    seq_idx_from_cu_seqlens_function,
)
from causal_conv1d_b200.torch_reference import causal_conv1d_varlen_states_ref  # noqa: F401


def causal_conv1d_varlen_states(x: Tensor, cu_seqlens: Tensor, state_len: int) -> Tensor:
    """
    Forward pass only, does not support backward pass.
    Parameters:
        x: (total_tokens, dim)
        cu_seqlens: (batch + 1), int32 or int64, sorted: cumulative sequence lengths from 0.
        state_len: how many trailing tokens of each sequence to copy into its state.
            Slots that would reach into the previous sequence are zero.
    Return:
        states: (batch, dim, state_len), stored channel-last (stride(1) == 1)
    """
    return causal_conv1d_varlen_states_function(x, cu_seqlens, state_len)


def seq_idx_from_cu_seqlens(cu_seqlens: Tensor, total_tokens: int) -> Tensor:
    """seq_idx (total_tokens,) int32: the sequence number of every packed token, -1 for tokens
    at or after ``cu_seqlens[-1]``.  (The reference's callers build this tensor with PyTorch
    ops, ``tests/test_causal_conv1d.py:437-447``.)"""
    return seq_idx_from_cu_seqlens_function(cu_seqlens, total_tokens)


def causal_conv1d_varlen_fn(
    x: Tensor,
    weight: Tensor,
    bias: Tensor | None = None,
    *,
    cu_seqlens: Tensor,
    seq_idx: Tensor | None = None,
    conv_states: Tensor | None = None,
    state_indices: Tensor | None = None,
    has_initial_state: Tensor | None = None,
    update_states: bool = True,
    activation: str | None = None,
) -> Tensor:
    """
    Packed variable-length prefill that continues from, and leaves behind, per-sequence conv
    states: one call for what the reference needs a per-sequence loop of
    ``causal_conv1d_fn(x_s, initial_states=..., return_final_states=True)``
    (``causal_conv1d/causal_conv1d_interface.py:99-129``; it forbids ``seq_idx`` together with
    states, ``:27-33``) plus ``causal_conv1d_varlen_states`` for. Forward only.

    Parameters:
        x: (total_tokens, dim), stride(1) == 1; sequence s owns rows cu_seqlens[s]:cu_seqlens[s+1]
        weight: (dim, width); bias: (dim,) or None
        cu_seqlens: (nseq + 1,) int32, from 0
        seq_idx: (total_tokens,) int32 or None (then built from cu_seqlens)
        conv_states: (rows, dim, state_len) with stride(1) == 1, state_len >= width - 1, or None.
            Row r = state_indices[s] (s when state_indices is None) holds sequence s's state.
        has_initial_state: (nseq,) bool or None.  Where True (everywhere when None and
            conv_states is given) the sequence's left context is the last width-1 entries of
            its row; elsewhere it is zeros.
        update_states: write each sequence's final state — the last state_len entries of
            [prefix | x_s] — back into its row of conv_states (in place).
        activation: None, "silu" or "swish"
    Return:
        out: (total_tokens, dim)
    """
    if activation not in [None, "silu", "swish"]:
        raise NotImplementedError("activation must be None, silu, or swish")
    return causal_conv1d_prefill_varlen_function(
        x, weight, bias, cu_seqlens, seq_idx, conv_states, state_indices, has_initial_state,
        update_states, activation in ["silu", "swish"])
