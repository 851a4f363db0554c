"""Host logic of the sharding wrapper with world_size-2 gloo ranks on CPU.  The per-shard
arithmetic is done by the CPU oracle (injected through ``bwd_impl``); what is under test is the
shard arithmetic, the packed gradient buffer and the single all-reduce."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_bwd(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight, dbias, dinit, silu):
    import oracle
    g = oracle.bwd(x, weight, bias, dout, seq_idx=seq_idx, initial_states=initial_states,
                   dfinal_states=dfinal_states, activation="silu" if silu else None)
    dx.copy_(g["dx"].to(dx.dtype))
    dweight.copy_(g["dweight"].float())
    if dbias is not None:
        dbias.copy_(g["dbias"].float())


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from causal_conv1d_b200.distributed import batch_shard, batch_sharded_backward, channel_shard
        torch.manual_seed(0)          # same full problem on every rank
        B, D, L, W = 5, 16, 37, 4     # 5 rows over 2 ranks: uneven shards
        x, dout = torch.randn(B, D, L), torch.randn(B, D, L)
        w, b = torch.randn(D, W), torch.randn(D)
        full = oracle.bwd(x, w, b, dout, activation="silu")
        dx, dw, db, _, packed = batch_sharded_backward(
            batch_shard(x, rank, world), w, b, batch_shard(dout, rank, world), activation="silu",
            bwd_impl=_oracle_bwd)
        assert packed.numel() == D * W + D and packed.dtype == torch.float32
        ok = torch.allclose(dw.double(), full["dweight"], rtol=1e-5, atol=1e-5)
        ok &= torch.allclose(db.double(), full["dbias"], rtol=1e-5, atol=1e-5)
        ok &= torch.allclose(dx.double(), batch_shard(full["dx"], rank, world), rtol=1e-6, atol=1e-6)
        # every rank ends with identical bits
        gathered = [torch.empty_like(packed) for _ in range(world)]
        dist.all_gather(gathered, packed)
        ok &= all(torch.equal(gathered[0], g) for g in gathered)
        # channel sharding: no communication, shards concatenate to the full result
        xs = channel_shard(x, rank, world)
        o = oracle.fwd(xs, channel_shard(w, rank, world, dim=0), channel_shard(b, rank, world, dim=0), activation="silu")
        ok &= torch.equal(o, channel_shard(oracle.fwd(x, w, b, activation="silu"), rank, world))
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_batch_sharded_backward_gloo():
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret.get(0) is True and ret.get(1) is True


def _oracle_fwd(x, weight, bias, seq_idx, initial_states, out, final_states_out, silu):
    import oracle
    out.copy_(oracle.fwd(x, weight, bias, seq_idx=seq_idx, initial_states=initial_states,
                         activation="silu" if silu else None).to(out.dtype))


def _oracle_bwd_states(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, dweight, dbias, dinit, silu):
    import oracle
    g = oracle.bwd(x, weight, bias, dout, seq_idx=seq_idx, initial_states=initial_states,
                   dfinal_states=dfinal_states, activation="silu" if silu else None)
    dx.copy_(g["dx"].to(dx.dtype))
    dweight.copy_(g["dweight"].float())
    if dbias is not None:
        dbias.copy_(g["dbias"].float())
    if dinit is not None:
        dinit.copy_(g["dinitial_states"].to(dinit.dtype))


def _seq_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from causal_conv1d_b200.distributed import (sequence_parallel_backward, sequence_parallel_forward,
                                                    sequence_shard)
        torch.manual_seed(1)          # same full problem on every rank
        B, D, L, W = 2, 8, 23, 4      # 23 tokens over 3 ranks: uneven shards
        x = torch.randn(B, L, D, dtype=torch.float64).transpose(1, 2)
        dout = torch.randn(B, L, D, dtype=torch.float64).transpose(1, 2)
        ini = torch.randn(B, W - 1, D, dtype=torch.float64).transpose(1, 2)
        w, b = torch.randn(D, W, dtype=torch.float64), torch.randn(D, dtype=torch.float64)
        full_out = oracle.fwd(x, w, b, initial_states=ini, activation="silu")
        full = oracle.bwd(x, w, b, dout, initial_states=ini, activation="silu")
        xs, ds = sequence_shard(x, rank, world), sequence_shard(dout, rank, world)
        out, halo = sequence_parallel_forward(xs, w, b, "silu", initial_states=ini if rank == 0 else None,
                                              fwd_impl=_oracle_fwd)
        ok = torch.allclose(out, sequence_shard(full_out, rank, world), rtol=1e-12, atol=1e-12)
        dx, dw, db, dini = sequence_parallel_backward(xs, w, b, ds, halo, "silu", return_dinitial_states=True,
                                                      bwd_impl=_oracle_bwd_states)
        ok &= torch.allclose(dx, sequence_shard(full["dx"], rank, world), rtol=1e-12, atol=1e-12)
        # weight gradients travel as fp32
        ok &= torch.allclose(dw, full["dweight"], rtol=1e-5, atol=1e-5) and torch.allclose(db, full["dbias"], rtol=1e-5, atol=1e-5)
        if rank == 0:
            ok &= torch.allclose(dini, full["dinitial_states"], rtol=1e-12, atol=1e-12)
        else:
            ok &= dini is None
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sequence_parallel_gloo():
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ret = mp.Manager().dict()
    mp.spawn(_seq_worker, args=(3, port, ret), nprocs=3, join=True)
    assert all(ret.get(r) is True for r in range(3))


def test_shard_bounds():
    from causal_conv1d_b200.distributed import channel_shard, shard_bounds
    assert [shard_bounds(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    t = torch.zeros(2, 5376, 3)
    widths = [channel_shard(t, r, 8).shape[1] for r in range(8)]
    assert sum(widths) == 5376 and all(w % 8 == 0 for w in widths)
    with pytest.raises(ValueError):
        channel_shard(torch.zeros(1, 12, 1), 0, 2)
