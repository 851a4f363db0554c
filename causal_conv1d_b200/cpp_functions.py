"""torch.library custom ops and allocating wrappers over the native extension.

Mirrors ``causal_conv1d/cpp_functions.py:8-183`` of the reference: three mutating ops that
return nothing, plus ``causal_conv1d_{fwd,bwd,update}_function`` which allocate outputs.
The ops live in their own library namespace so that this package and a reference build can
be loaded in one process.  In eager mode the wrappers call the extension directly (the
custom-op dispatcher costs more than a decode-step kernel); under ``torch.compile`` they go
through the registered ops.
"""
import torch

from causal_conv1d_b200._ext import ext as _ext

LIBRARY_NAME = "cc1d_b200"


@torch.library.custom_op(f"{LIBRARY_NAME}::_causal_conv1d_fwd_cpp", mutates_args={"out", "final_states_out"})
def _causal_conv1d_fwd_cpp(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    seq_idx: torch.Tensor | None,
    initial_states: torch.Tensor | None,
    out: torch.Tensor,
    final_states_out: torch.Tensor | None,
    silu_activation: bool,
) -> None:
    _ext.causal_conv1d_fwd(x, weight, bias, seq_idx, initial_states, out, final_states_out, silu_activation)


@torch.library.custom_op(
    f"{LIBRARY_NAME}::_causal_conv1d_bwd_cpp",
    mutates_args={"dfinal_states", "dx", "dweight", "dbias", "dinitial_states"},
)
def _causal_conv1d_bwd_cpp(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    dout: torch.Tensor,
    seq_idx: torch.Tensor | None,
    initial_states: torch.Tensor | None,
    dfinal_states: torch.Tensor | None,
    dx: torch.Tensor,
    dweight: torch.Tensor,
    dbias: torch.Tensor | None,
    dinitial_states: torch.Tensor | None,
    silu_activation: bool,
) -> None:
    # dweight / dbias are fully overwritten (fixed-order reduction, no atomics)
    _ext.causal_conv1d_bwd(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight, dbias,
                           dinitial_states, silu_activation, False)


@torch.library.custom_op(f"{LIBRARY_NAME}::_causal_conv1d_update_cpp", mutates_args={"out", "conv_state"})
def _causal_conv1d_update_cpp(
    x: torch.Tensor,
    conv_state: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    out: torch.Tensor,
    silu_activation: bool,
    cache_seqlens: torch.Tensor | None,
    conv_state_indices: torch.Tensor | None,
) -> None:
    _ext.causal_conv1d_update(x, conv_state, weight, bias, out, silu_activation, cache_seqlens, conv_state_indices)


@torch.library.custom_op(f"{LIBRARY_NAME}::_causal_conv1d_varlen_states_cpp", mutates_args={"states"})
def _causal_conv1d_varlen_states_cpp(x: torch.Tensor, cu_seqlens: torch.Tensor, states: torch.Tensor) -> None:
    _ext.causal_conv1d_varlen_states(x, cu_seqlens, states)


def _compiling() -> bool:
    return torch.compiler.is_compiling()


def causal_conv1d_fwd_function(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    seq_idx: torch.Tensor | None,
    initial_states: torch.Tensor | None,
    final_states_out: torch.Tensor | None,
    silu_activation: bool,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``out`` (not in the reference's signature): a caller-provided result buffer of x's shape,
    dtype and layout class with any batch / row strides — e.g. a slice of the buffer the next
    op reads — the forward counterpart of the ``dx`` hook of the backward wrapper
    (``causal_conv1d/cpp_functions.py:125,132``).  Saves the copy a caller would otherwise make."""
    if out is None:
        out = torch.empty_like(x)
    fn = _causal_conv1d_fwd_cpp if _compiling() else _ext.causal_conv1d_fwd
    fn(x, weight, bias, seq_idx, initial_states, out, final_states_out, silu_activation)
    return out


def causal_conv1d_bwd_function(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    dout: torch.Tensor,
    seq_idx: torch.Tensor | None,
    initial_states: torch.Tensor | None,
    dfinal_states: torch.Tensor | None,
    dx: torch.Tensor | None,
    return_dinitial_states: bool,
    silu_activation: bool,
) -> tuple[torch.Tensor | None]:
    batch_size, dim = x.size()[:2]
    width = weight.size(-1)
    if dx is None:
        dx = torch.empty_like(x)
    # The reference zero-fills these for its atomics (cpp_functions.py:134-137); here the
    # kernels overwrite them, so no memset is needed.
    dweight = torch.empty_like(weight, dtype=torch.float32)
    dbias = torch.empty_like(bias, dtype=torch.float32) if bias is not None else None
    dinitial_states = None
    if return_dinitial_states:
        dinitial_states = torch.empty(batch_size, width - 1, dim, device=x.device, dtype=x.dtype).transpose(1, 2)
    if _compiling():
        _causal_conv1d_bwd_cpp(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight, dbias,
                               dinitial_states, silu_activation)
    else:
        _ext.causal_conv1d_bwd(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight, dbias,
                               dinitial_states, silu_activation, False)
    dweight = dweight.type_as(weight)
    if dbias is not None:
        dbias = dbias.type_as(bias)
    return dx, dweight, dbias, dinitial_states


def causal_conv1d_update_function(
    x: torch.Tensor,
    conv_state: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    silu_activation: bool,
    cache_seqlens: torch.Tensor | None,
    conv_state_indices: torch.Tensor | None,
) -> torch.Tensor:
    out = torch.empty_like(x)
    fn = _causal_conv1d_update_cpp if _compiling() else _ext.causal_conv1d_update
    fn(x, conv_state, weight, bias, out, silu_activation, cache_seqlens, conv_state_indices)
    return out


def causal_conv1d_varlen_states_function(x: torch.Tensor, cu_seqlens: torch.Tensor, state_len: int) -> torch.Tensor:
    _, dim = x.shape
    batch = cu_seqlens.shape[0] - 1
    states = torch.empty(batch, state_len, dim, dtype=x.dtype, device=x.device).transpose(1, 2)
    fn = _causal_conv1d_varlen_states_cpp if _compiling() else _ext.causal_conv1d_varlen_states
    fn(x, cu_seqlens.contiguous(), states)
    return states


def seq_idx_from_cu_seqlens_function(cu_seqlens: torch.Tensor, total_tokens: int) -> torch.Tensor:
    seq_idx = torch.empty(total_tokens, dtype=torch.int32, device=cu_seqlens.device)
    _ext.seq_idx_from_cu_seqlens(cu_seqlens.to(torch.int32).contiguous(), seq_idx)
    return seq_idx


def causal_conv1d_prefill_varlen_function(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    cu_seqlens: torch.Tensor,
    seq_idx: torch.Tensor | None,
    conv_states: torch.Tensor | None,
    state_indices: torch.Tensor | None,
    has_initial_state: torch.Tensor | None,
    update_states: bool,
    silu_activation: bool,
) -> torch.Tensor:
    """Packed varlen prefill continuing from / updating per-sequence conv states; eager only
    (no custom op is registered for it)."""
    cu = cu_seqlens.to(torch.int32).contiguous()
    if seq_idx is None:
        seq_idx = seq_idx_from_cu_seqlens_function(cu, x.shape[0])
    out = torch.empty_like(x)
    if has_initial_state is not None:
        has_initial_state = has_initial_state.to(torch.bool).contiguous()
    if state_indices is not None:
        state_indices = state_indices.to(torch.int32).contiguous()
    _ext.causal_conv1d_prefill_varlen(
        x, weight, bias, seq_idx.reshape(-1), cu,
        conv_states,
        conv_states if (conv_states is not None and update_states) else None,
        state_indices, has_initial_state, out, silu_activation)
    return out
