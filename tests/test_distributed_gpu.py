"""Batch-sharded backward, channel-sharded decode and the sequence-parallel hand-off on 2 real
GPUs (NCCL).  Skipped when
fewer than 2 devices are visible."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from causal_conv1d_b200 import causal_conv1d_update
        from causal_conv1d_b200.distributed import batch_shard, batch_sharded_backward, channel_shard
        torch.manual_seed(0)   # the same full problem on every rank
        B, D, L, W = 6, 256, 1000, 4
        x = torch.randn(B, D, L, dtype=torch.bfloat16).to(dev)
        dout = torch.randn(B, D, L, dtype=torch.bfloat16).to(dev)
        w, b = torch.randn(D, W).to(dev), torch.randn(D).to(dev)
        # unsharded result on this GPU
        full = batch_sharded_backward(x, w, b, dout, activation="silu", group=dist.new_group([rank]))
        dx, dw, db, _, packed = batch_sharded_backward(batch_shard(x, rank, world), w, b, batch_shard(dout, rank, world),
                                                       activation="silu")
        ok = torch.equal(dx, batch_shard(full[0], rank, world))                 # dx needs no communication
        ok &= torch.allclose(dw, full[1], rtol=1e-5, atol=1e-4) and torch.allclose(db, full[2], rtol=1e-5, atol=1e-4)
        gathered = [torch.empty_like(packed) for _ in range(world)]
        dist.all_gather(gathered, packed)
        ok &= all(torch.equal(gathered[0], g) for g in gathered)                # every rank holds the same bits
        # channel-sharded decode: shards of x / state / weight, no collective
        xs = torch.randn(8, D, dtype=torch.bfloat16).to(dev)
        st = torch.randn(8, 3, D, dtype=torch.bfloat16).to(dev).transpose(1, 2)
        st_full = st.clone()
        out_full = causal_conv1d_update(xs, st_full, w, b, activation="silu")
        st_sh = channel_shard(st, rank, world).contiguous().transpose(1, 2).contiguous().transpose(1, 2)
        out_sh = causal_conv1d_update(channel_shard(xs, rank, world).contiguous(), st_sh, channel_shard(w, rank, world, dim=0),
                                      channel_shard(b, rank, world, dim=0), activation="silu")
        ok &= torch.equal(out_sh, channel_shard(out_full, rank, world)) and torch.equal(st_sh, channel_shard(st_full, rank, world))
        # sequence parallel: halo hand-off as initial_states, dinitial_states folded back into dx
        from causal_conv1d_b200 import causal_conv1d_fn
        from causal_conv1d_b200.distributed import (sequence_parallel_backward, sequence_parallel_forward,
                                                    sequence_shard)
        xl = torch.randn(2, 777, D, dtype=torch.bfloat16).to(dev).transpose(1, 2)
        dl = torch.randn(2, 777, D, dtype=torch.bfloat16).to(dev).transpose(1, 2)
        xr = xl.detach().clone().requires_grad_()
        wr, br = w.clone().requires_grad_(), b.clone().requires_grad_()
        out_full = causal_conv1d_fn(xr, wr, br, activation="silu")
        out_full.backward(dl)
        xs, dsh = sequence_shard(xl, rank, world), sequence_shard(dl, rank, world)
        out_s, halo = sequence_parallel_forward(xs, w, b, "silu")
        ok &= torch.equal(out_s, sequence_shard(out_full, rank, world))          # same arithmetic, same bits
        dx_s, dw_s, db_s, _ = sequence_parallel_backward(xs, w, b, dsh, halo, "silu")
        ref_dx = sequence_shard(xr.grad, rank, world)
        ok &= torch.equal(dx_s[:, :, : -(W - 1)], ref_dx[:, :, : -(W - 1)])      # away from the seam: identical
        seam = (dx_s[:, :, -(W - 1):].float() - ref_dx[:, :, -(W - 1):].float()).abs()
        ok &= bool((seam <= 1e-2 * ref_dx[:, :, -(W - 1):].float().abs().clamp(min=1.0)).all())
        ok &= torch.allclose(dw_s, wr.grad, rtol=1e-5, atol=1e-4) and torch.allclose(db_s, br.grad, rtol=1e-5, atol=1e-4)
        # one-shot all-reduce over peer memory against NCCL, several epochs (both parities)
        from causal_conv1d_b200.distributed import PeerGradReducer
        red = PeerGradReducer(D * W + D)
        for step in range(5):
            torch.manual_seed(100 + step * world + rank)
            part = torch.randn(D * W + D, device=dev)
            want = part.clone()
            dist.all_reduce(want)
            got = red.reduce_(part.clone())
            ok &= torch.allclose(got, want, rtol=1e-6, atol=1e-6)
            both = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(both, got)
            ok &= all(torch.equal(both[0], g) for g in both)                     # same bits on every rank
        red.check()
        dx_p, dw_p, db_p, _, _ = batch_sharded_backward(batch_shard(x, rank, world), w, b, batch_shard(dout, rank, world),
                                                        activation="silu", reducer=red)
        ok &= torch.equal(dx_p, dx) and torch.allclose(dw_p, dw, rtol=1e-6, atol=1e-6) and torch.allclose(db_p, db, rtol=1e-6, atol=1e-6)
        red.check()
        # the same exchange inside the backward's finishing kernel: one kernel less, same bits as the two-kernel path
        fused = PeerGradReducer(D * W + D, fused=True)
        for _ in range(3):
            dx_f, dw_f, db_f, _, packed_f = batch_sharded_backward(batch_shard(x, rank, world), w, b, batch_shard(dout, rank, world),
                                                                   activation="silu", reducer=fused)
            ok &= torch.equal(dx_f, dx) and torch.equal(dw_f, dw_p) and torch.equal(db_f, db_p)
        fused.check()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharding():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret.get(0) is True and ret.get(1) is True


def test_one_process_two_devices():
    """One process driving two GPUs: per-device set-up inside the library (the shared-memory
    opt-in of the TMA kernels, the occupancy cache) must hold on the second device too."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    sys.path.insert(0, ROOT)
    from causal_conv1d_b200 import causal_conv1d_fn
    torch.manual_seed(0)
    x0 = torch.randn(2, 700, 256, dtype=torch.bfloat16)
    w0, b0 = torch.randn(256, 4), torch.randn(256)
    res = []
    for d in (0, 1, 0):
        dev = torch.device("cuda", d)
        x = x0.to(dev).transpose(1, 2).requires_grad_()        # channel-last: TMA kernels
        w, b = w0.to(dev).requires_grad_(), b0.to(dev).requires_grad_()
        out = causal_conv1d_fn(x, w, b, activation="silu")
        out.backward(torch.ones_like(out))
        torch.cuda.synchronize(dev)
        res.append((out.detach().cpu(), x.grad.cpu(), w.grad.cpu(), b.grad.cpu()))
    for r in res[1:]:
        assert all(torch.equal(a, c) for a, c in zip(res[0], r))


def _peer_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from causal_conv1d_b200.distributed import PeerGradReducer
        ok = True
        for count in (25600, 26880, 1000):          # C2 and C3 gradient buffers, and one that needs staging
            red = PeerGradReducer(count)
            for step in range(4):
                torch.manual_seed(7 * step + rank)
                part = torch.randn(count, device=dev)
                want = part.clone()
                dist.all_reduce(want)
                got = red.reduce_(part.clone())
                ok &= torch.allclose(got, want, rtol=1e-5, atol=1e-5)
                every = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(every, got)
                ok &= all(torch.equal(every[0], g) for g in every)
                # the fixed rank order of the additions, reproduced on the host
                parts = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(parts, part)
                acc = parts[0].clone()
                for p in parts[1:]:
                    acc += p
                ok &= torch.equal(got, acc)
            red.check()
        # the batch-sharded backward on all ranks: exchange inside the finishing kernel against NCCL
        from causal_conv1d_b200.distributed import batch_shard, batch_sharded_backward
        torch.manual_seed(0)
        B, D, L, W = 2 * world, 136, 1024, 4
        x = torch.randn(B, D, L, dtype=torch.bfloat16).to(dev)
        dout = torch.randn(B, D, L, dtype=torch.bfloat16).to(dev)
        w, b = torch.randn(D, W).to(dev), torch.randn(D).to(dev)
        xs, ds = batch_shard(x, rank, world), batch_shard(dout, rank, world)
        dx_n, dw_n, db_n, _, _ = batch_sharded_backward(xs, w, b, ds, activation="silu")
        fused = PeerGradReducer(D * W + D, fused=True)
        for _ in range(3):                           # both parities of the exchange buffer
            dx_f, dw_f, db_f, _, packed = batch_sharded_backward(xs, w, b, ds, activation="silu", reducer=fused)
            ok &= torch.equal(dx_f, dx_n)
            ok &= torch.allclose(dw_f, dw_n, rtol=1e-5, atol=1e-4) and torch.allclose(db_f, db_n, rtol=1e-5, atol=1e-4)
            every = [torch.empty_like(packed) for _ in range(world)]
            dist.all_gather(every, packed)
            ok &= all(torch.equal(every[0], g) for g in every)
        fused.check()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_peer_allreduce_on_all_visible_gpus():
    """As many ranks as there are GPUs (2 to 8): same result as NCCL within fp32 rounding, the
    same bits on every rank, and exactly the sum taken in rank order; then the batch-sharded
    backward with the exchange fused into its finishing kernel."""
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs 2 GPUs")
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ret = mp.Manager().dict()
    mp.spawn(_peer_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) is True for r in range(world))
