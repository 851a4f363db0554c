"""``causal_conv1d_varlen_states`` — same signature as the reference's Triton-backed
function (``causal_conv1d/causal_conv1d_varlen.py:35-64``), served by a CUDA kernel."""
from torch import Tensor

from causal_conv1d_b200.cpp_functions import causal_conv1d_varlen_states_function


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
