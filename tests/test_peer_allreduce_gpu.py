"""cc1d_peer_allreduce on ONE GPU: the buffer layout, the flag protocol and the bounded wait,
without two kernels ever waiting for each other (the real two-GPU run is in
test_distributed_gpu.py).  Ranks are emulated by separate exchange buffers on the same device;
data a not-yet-run "peer" would have delivered is put there by hand."""
import pytest
import torch

pytestmark = pytest.mark.gpu

FLAG_BYTES, MAX_PEERS, CTAS = 4096, 16, 8


def _ext():
    from causal_conv1d_b200._ext import ext
    return ext


def _buffer(world, count):
    n = _ext().peer_allreduce_buffer_bytes(world, count)
    assert n == FLAG_BYTES + 2 * world * count * 4
    return torch.zeros(n // 4, dtype=torch.float32, device="cuda")


def _deliver(buf, world, count, parity, from_rank, vec, epoch):
    """What rank `from_rank`'s kernel leaves in a peer's exchange buffer."""
    slots = buf[FLAG_BYTES // 4:].view(2, world, count)
    slots[parity, from_rank] = vec
    flags = buf[:FLAG_BYTES // 4].view(torch.int32)[: 2 * MAX_PEERS * CTAS].view(2, MAX_PEERS, CTAS)
    flags[parity, from_rank] = epoch


@pytest.mark.parametrize("count", [4, 1000, 25600, 40964])
def test_world_of_one_is_identity(count):
    ext = _ext()
    buf, status = _buffer(1, count), torch.zeros(1, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):
        v = torch.randn(count, device="cuda")
        want = v.clone()
        ext.peer_allreduce(v, [buf.data_ptr()], 0, epoch, status)
        assert torch.equal(v, want)
    assert int(status.item()) == 0


def test_two_ranks_emulated_on_one_device():
    ext = _ext()
    torch.manual_seed(0)
    world, count = 2, 25600
    bufs = [_buffer(world, count), _buffer(world, count)]
    ptrs = [b.data_ptr() for b in bufs]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3, 4):
        parts = [torch.randn(count, device="cuda") for _ in range(world)]
        want = parts[0] + parts[1]                      # rank order 0, 1
        # rank 1 runs first; rank 0's contribution to rank 1's buffer is delivered by hand
        _deliver(bufs[1], world, count, epoch & 1, 0, parts[0], epoch)
        got1 = parts[1].clone()
        ext.peer_allreduce(got1, ptrs, 1, epoch, status)
        # rank 1's kernel has written its slice and flags into rank 0's buffer: rank 0 finds them
        got0 = parts[0].clone()
        ext.peer_allreduce(got0, ptrs, 0, epoch, status)
        assert torch.equal(got0, want) and torch.equal(got1, want), f"epoch {epoch}"
    assert int(status.item()) == 0


def test_wait_runs_out_instead_of_hanging():
    """A peer that never delivers: the kernel gives up after its bounded wait (about half a
    second), raises the status word and leaves the destination untouched."""
    ext = _ext()
    world, count = 2, 1024
    bufs = [_buffer(world, count), _buffer(world, count)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    v = torch.randn(count, device="cuda")
    keep = v.clone()
    ext.peer_allreduce(v, [b.data_ptr() for b in bufs], 0, 1, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert torch.equal(v, keep)
    # the context is still usable and the next collective works once the peer does deliver
    status.zero_()
    _deliver(bufs[0], world, count, 0, 1, torch.ones(count, device="cuda"), 2)
    ext.peer_allreduce(v, [b.data_ptr() for b in bufs], 0, 2, status)
    assert int(status.item()) == 0 and torch.equal(v, keep + 1)


def test_rejects_bad_arguments():
    ext = _ext()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    buf = _buffer(1, 8)
    with pytest.raises(RuntimeError):
        ext.peer_allreduce(torch.zeros(6, device="cuda"), [buf.data_ptr()], 0, 1, status)      # count % 4
    with pytest.raises(RuntimeError):
        ext.peer_allreduce(torch.zeros(8, device="cuda"), [buf.data_ptr()], 0, 0, status)      # epoch 0
    with pytest.raises(RuntimeError):
        ext.peer_allreduce(torch.zeros(8, device="cuda"), [buf.data_ptr()], 1, 1, status)      # rank >= world
