"""Sharding helpers for one process per GPU (``torch.distributed``).

The op is independent per (batch, channel) row, so forward, decode update and varlen
states need no communication under either sharding.  The only exchange is in the
batch-sharded backward: every rank holds a partial ``dweight`` / ``dbias`` (sums over its
own batch rows); they are packed into ONE fp32 buffer ``[dim * width + dim]`` and summed
with a single all-reduce, in fp32 and before the cast to the weight dtype, so that the
result does not depend on the number of ranks beyond fp32 rounding.

The reference has no distributed code; this module is the multi-GPU wrapper the hot path
needs.  Nothing here reads another GPU's memory directly.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def shard_bounds(n: int, rank: int, world_size: int) -> tuple[int, int]:
    """Contiguous, balanced split of range(n): first ``n % world_size`` ranks get one extra."""
    base, extra = divmod(n, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def batch_shard(t: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    lo, hi = shard_bounds(t.shape[0], rank, world_size)
    return t[lo:hi]


def channel_shard(t: torch.Tensor, rank: int, world_size: int, dim: int = 1, multiple_of: int = 8) -> torch.Tensor:
    """Slice the channel dimension; shard edges fall on multiples of ``multiple_of`` so that
    every shard keeps the channel-last alignment rule (dim % 8 == 0)."""
    n = t.shape[dim]
    if n % multiple_of:
        raise ValueError(f"channel count {n} is not a multiple of {multiple_of}")
    lo, hi = shard_bounds(n // multiple_of, rank, world_size)
    return t.narrow(dim, lo * multiple_of, (hi - lo) * multiple_of)


def packed_grad_buffer(dim: int, width: int, has_bias: bool, device) -> tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """One fp32 allocation viewed as dweight (dim, width) and dbias (dim,): the all-reduce
    payload, written in place by the backward kernels."""
    packed = torch.empty(dim * width + (dim if has_bias else 0), dtype=torch.float32, device=device)
    dweight = packed[: dim * width].view(dim, width)
    dbias = packed[dim * width:] if has_bias else None
    return packed, dweight, dbias


def _default_bwd():
    from causal_conv1d_b200._ext import ext

    def run(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight, dbias, dinitial_states, silu):
        ext.causal_conv1d_bwd(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight, dbias,
                              dinitial_states, silu, False)

    return run


def batch_sharded_backward(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    dout: torch.Tensor,
    activation: Optional[str] = None,
    seq_idx: Optional[torch.Tensor] = None,
    initial_states: Optional[torch.Tensor] = None,
    dfinal_states: Optional[torch.Tensor] = None,
    dx: Optional[torch.Tensor] = None,
    return_dinitial_states: bool = False,
    group: Optional[dist.ProcessGroup] = None,
    bwd_impl: Optional[Callable] = None,
):
    """Backward of this rank's batch shard followed by the single all-reduce of the packed
    fp32 weight gradients.  ``x`` / ``dout`` / states are the LOCAL shards; weight and bias
    are replicated.  Returns (dx, dweight, dbias, dinitial_states, packed_fp32) with
    dweight/dbias cast to the weight dtype after the reduction.

    ``bwd_impl`` exists for the CPU (gloo) tests of this host logic; the default is the
    CUDA extension.
    """
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    run = bwd_impl if bwd_impl is not None else _default_bwd()
    dim, width = weight.shape
    if dx is None:
        dx = torch.empty_like(x)
    packed, dweight32, dbias32 = packed_grad_buffer(dim, width, bias is not None, x.device)
    dinit = None
    if return_dinitial_states:
        dinit = torch.empty(x.shape[0], width - 1, dim, device=x.device, dtype=x.dtype).transpose(1, 2)
    run(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight32, dbias32, dinit,
        activation is not None)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    dweight = dweight32.to(weight.dtype)
    dbias = dbias32.to(bias.dtype) if bias is not None else None
    return dx, dweight, dbias, dinit, packed
