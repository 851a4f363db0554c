"""Sharding helpers for one process per GPU (``torch.distributed``).

The op is independent per (batch, channel) row, so forward, decode update and varlen
states need no communication under either sharding.  The only exchange is in the
batch-sharded backward: every rank holds a partial ``dweight`` / ``dbias`` (sums over its
own batch rows); they are packed into ONE fp32 buffer ``[dim * width + dim]`` and summed
with a single all-reduce, in fp32 and before the cast to the weight dtype, so that the
result does not depend on the number of ranks beyond fp32 rounding.

The reference has no distributed code; this module is the multi-GPU wrapper the hot path
needs.  Nothing here reads another GPU's memory; ``PeerGradReducer`` writes into peers' buffers.
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

    def run(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight, dbias, dinitial_states, silu, **peer):
        ext.causal_conv1d_bwd(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight, dbias,
                              dinitial_states, silu, False, **peer)

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
    reducer: Optional["PeerGradReducer"] = None,
):
    """Backward of this rank's batch shard followed by the single all-reduce of the packed
    fp32 weight gradients (NCCL/gloo ``all_reduce``; ``reducer.reduce_`` when a
    ``PeerGradReducer`` is given; inside the backward's own finishing kernel when that reducer
    was created with ``fused=True``).  ``x`` / ``dout`` / states are the LOCAL shards; weight and bias
    are replicated.  Returns (dx, dweight, dbias, dinitial_states, packed_fp32) with
    dweight/dbias cast to the weight dtype after the reduction.  With a ``reducer`` the wait for
    the other ranks is bounded: if it ran out the gradients are NaN and ``reducer.check()``
    raises — call it before the optimizer step.

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
    fused = reducer is not None and reducer.fused
    if fused and bwd_impl is not None:
        raise ValueError("a fused reducer needs the CUDA extension's backward")
    run(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight32, dbias32, dinit,
        activation is not None, **(reducer.backward_args() if fused else {}))
    if fused:
        pass                                 # dweight32 / dbias32 already hold the sum over all ranks
    elif reducer is not None:
        reducer.reduce_(packed)
    elif dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    dweight = dweight32.to(weight.dtype)
    dbias = dbias32.to(bias.dtype) if bias is not None else None
    return dx, dweight, dbias, dinit, packed


# ---- sequence (context) parallel: the sequence axis is split across ranks ---------------------
#
# Rank r holds tokens [lo_r, hi_r) of every (batch, channel) row, channel-last.  The conv at the
# first width-1 tokens of a shard needs the last width-1 tokens of the previous shard: each rank
# sends that tail to rank r+1, which takes it as ``initial_states`` — the hook the reference has
# for chunked processing (``causal_conv1d/causal_conv1d_interface.py:99-129``).  Because the
# tail is raw input (not a conv result) all ranks run concurrently: one neighbour exchange of
# batch * dim * (width-1) elements, then the ordinary forward.  In the backward the gradient
# that rank r+1 computes for its ``initial_states`` belongs to the last width-1 tokens of rank
# r's dx: one neighbour exchange the other way and an add on that slice, then the same packed
# all-reduce of dweight / dbias as in the batch-sharded case.

def sequence_shard(t: torch.Tensor, rank: int, world_size: int, dim: int = 2) -> torch.Tensor:
    lo, hi = shard_bounds(t.shape[dim], rank, world_size)
    return t.narrow(dim, lo, hi - lo)


def _neighbour_exchange(send: Optional[torch.Tensor], recv: Optional[torch.Tensor], send_to: int, recv_from: int,
                        group) -> None:
    """Post at most one send and one receive and wait for both."""
    ops = []
    if send is not None:
        ops.append(dist.P2POp(dist.isend, send, send_to, group))
    if recv is not None:
        ops.append(dist.P2POp(dist.irecv, recv, recv_from, group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()


def _default_fwd():
    from causal_conv1d_b200._ext import ext

    def run(x, weight, bias, seq_idx, initial_states, out, final_states_out, silu):
        ext.causal_conv1d_fwd(x, weight, bias, seq_idx, initial_states, out, final_states_out, silu)

    return run


def _state_buffer(batch: int, dim: int, width: int, like: torch.Tensor) -> torch.Tensor:
    """(batch, dim, width-1) with stride(1) == 1, the layout the kernels take for states."""
    return torch.empty(batch, width - 1, dim, device=like.device, dtype=like.dtype).transpose(1, 2)


def sequence_parallel_forward(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    activation: Optional[str] = None,
    initial_states: Optional[torch.Tensor] = None,
    group: Optional[dist.ProcessGroup] = None,
    fwd_impl: Optional[Callable] = None,
):
    """Forward of this rank's sequence shard ``x`` (batch, dim, local_len), channel-last
    (``x.stride(1) == 1``), local_len >= width - 1 on every rank.  ``initial_states`` is the
    left context of the whole sequence and is read on rank 0 only.
    Returns (out, halo): ``halo`` is the left context this rank used (None on rank 0 without
    initial_states); keep it for ``sequence_parallel_backward``."""
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    run = fwd_impl if fwd_impl is not None else _default_fwd()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    batch, dim, seqlen = x.shape
    width = weight.shape[1]
    if seqlen < width - 1:
        raise ValueError("every sequence shard must hold at least width - 1 tokens")
    halo = initial_states if rank == 0 else _state_buffer(batch, dim, width, x)
    tail = None
    if rank + 1 < world:
        tail = _state_buffer(batch, dim, width, x)
        tail.copy_(x[:, :, seqlen - (width - 1):])
    if world > 1:
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
        _neighbour_exchange(tail.transpose(1, 2) if tail is not None else None,
                            halo.transpose(1, 2) if rank > 0 else None,
                            ranks[min(rank + 1, world - 1)], ranks[max(rank - 1, 0)], group)
    out = torch.empty_like(x)
    run(x, weight, bias, None, halo, out, None, activation is not None)
    return out, halo


def sequence_parallel_backward(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    dout: torch.Tensor,
    halo: Optional[torch.Tensor],
    activation: Optional[str] = None,
    return_dinitial_states: bool = False,
    group: Optional[dist.ProcessGroup] = None,
    bwd_impl: Optional[Callable] = None,
):
    """Backward of this rank's sequence shard.  Returns (dx, dweight, dbias, dinitial_states):
    dweight / dbias are the sums over all shards (one all-reduce of the packed fp32 buffer);
    dinitial_states is the gradient of the whole sequence's left context, on rank 0 when asked.
    The last width-1 positions of dx are the sum of two terms rounded separately to the I/O
    dtype (this rank's taps, the next rank's taps)."""
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    run = bwd_impl if bwd_impl is not None else _default_bwd()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    batch, dim, seqlen = x.shape
    width = weight.shape[1]
    dx = torch.empty_like(x)
    packed, dweight32, dbias32 = packed_grad_buffer(dim, width, bias is not None, x.device)
    want_dhalo = halo is not None and (rank > 0 or return_dinitial_states)
    dhalo = _state_buffer(batch, dim, width, x) if want_dhalo else None
    run(x, weight, bias, dout, None, halo, None, dx, dweight32, dbias32, dhalo, activation is not None)
    if world > 1:
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
        from_next = _state_buffer(batch, dim, width, x) if rank + 1 < world else None
        _neighbour_exchange(dhalo.transpose(1, 2) if rank > 0 else None,
                            from_next.transpose(1, 2) if from_next is not None else None,
                            ranks[max(rank - 1, 0)], ranks[min(rank + 1, world - 1)], group)
        if from_next is not None:
            dx[:, :, seqlen - (width - 1):] += from_next
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    dweight = dweight32.to(weight.dtype)
    dbias = dbias32.to(bias.dtype) if bias is not None else None
    return dx, dweight, dbias, (dhalo if rank == 0 and return_dinitial_states else None)


# ---- one-shot all-reduce of the packed gradient buffer over NVLink peer memory ------------------
class PeerGradReducer:
    """Sum of the packed fp32 gradient buffer over the ranks of ``group`` in ONE kernel per rank
    (``cc1d_peer_allreduce``): every rank stores its vector into every peer's exchange buffer
    over NVLink, flags it, waits (bounded) for the others and adds them in rank order — the same
    bits on every rank, a few microseconds instead of a ring's latency.  The exchange buffers are
    peer-mapped allocations of PyTorch's symmetric memory; only plain peer stores cross NVLink
    (no multicast, no peer loads).

    ``reduce_(buf)`` sums ``buf`` in place (float32, numel <= count).  A peer that never shows up
    makes the kernel give up after ``spin_limit`` polls of about 0.25 us each (0: the library's
    default, about half a second — size it to the largest skew the job can have between ranks:
    a first step that loads code lazily, a host stall, an evaluation on one rank).  Giving up
    sets a status word and leaves NaN in every sum that could not be completed, so the result
    cannot be used by accident; ``check()`` (synchronises) raises if it ever happened.  Call
    ``check()`` before anything that cannot be undone, such as the optimizer step.
    """

    def __init__(self, count: int, group: Optional[dist.ProcessGroup] = None, device=None, fused: bool = False,
                 spin_limit: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        from causal_conv1d_b200._ext import ext

        self._ext = ext
        # fused: the exchange happens inside the backward's finishing kernel (see
        # batch_sharded_backward); the buffer then belongs to that kernel and reduce_ is not available
        self.fused = bool(fused)
        self.spin_limit = int(spin_limit)
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.count = (int(count) + 3) // 4 * 4
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        nbytes = ext.peer_allreduce_buffer_bytes(self.world, self.count)
        self._exchange = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=device)
        self._exchange.zero_()
        self._handle = symm_mem.rendezvous(self._exchange, self.group)
        self._peer_ptrs = [int(p) for p in self._handle.buffer_ptrs]
        self._staging = torch.zeros(self.count, dtype=torch.float32, device=device)
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)          # every rank's buffer is zeroed before anyone writes into it

    def backward_args(self) -> dict:
        """Keyword arguments that make ``ext.causal_conv1d_bwd`` sum dweight / dbias over the ranks."""
        if not self.fused:
            raise RuntimeError("this reducer was not created with fused=True")
        return dict(peer_ptrs=self._peer_ptrs, peer_rank=self.rank, peer_capacity=self.count, peer_status=self._status,
                    peer_spin_limit=self.spin_limit)

    def reduce_(self, buf: torch.Tensor) -> torch.Tensor:
        if self.fused:
            raise RuntimeError("a fused reducer exchanges inside the backward kernel; use batch_sharded_backward")
        n = buf.numel()
        if buf.dtype != torch.float32 or n > self.count:
            raise ValueError("buf must be float32 with at most `count` elements")
        direct = n == self.count and buf.is_contiguous() and buf.data_ptr() % 16 == 0
        work = buf if direct else self._staging
        if not direct:
            work[:n].copy_(buf.reshape(-1))
        # epoch 0: the kernel numbers the collectives itself, so the call can be replayed in a CUDA graph
        self._ext.peer_allreduce(work, self._peer_ptrs, self.rank, 0, self._status, self.spin_limit)
        if not direct:
            buf.copy_(work[:n].view_as(buf))
        return buf

    def check(self) -> None:
        if int(self._status.item()) != 0:
            raise RuntimeError("cc1d_peer_allreduce: a rank did not arrive within the wait limit")
