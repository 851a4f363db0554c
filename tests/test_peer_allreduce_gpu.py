"""cc1d_peer_allreduce on ONE GPU: the buffer layout, the flag protocol and the bounded wait,
without two kernels ever waiting for each other (the real two-GPU run is in
test_distributed_gpu.py).  Ranks are emulated by separate exchange buffers on the same device;
data a not-yet-run "peer" would have delivered is put there by hand."""
import pytest
import torch

pytestmark = pytest.mark.gpu

HEADER_BYTES, CTAS = 4096, 8


def _ext():
    from causal_conv1d_b200._ext import ext
    return ext


def _buffer(world, count):
    n = _ext().peer_allreduce_buffer_bytes(world, count)
    assert n == HEADER_BYTES + 2 * world * count * 8      # 16-byte lines of two values and two stamps
    return torch.zeros(n // 4, dtype=torch.float32, device="cuda")


def _deliver(buf, world, count, parity, from_rank, vec, epoch):
    """What rank `from_rank`'s kernel leaves in a peer's exchange buffer."""
    lines = buf[HEADER_BYTES // 4:].view(torch.int32).view(2, world, count // 2, 4)
    lines[parity, from_rank, :, 0] = vec[0::2].view(torch.int32)
    lines[parity, from_rank, :, 2] = vec[1::2].view(torch.int32)
    lines[parity, from_rank, :, 1] = epoch
    lines[parity, from_rank, :, 3] = epoch


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


def test_device_side_epoch_and_graph_replay():
    """epoch 0: the kernel counts the collectives itself, so a captured graph can be replayed."""
    ext = _ext()
    count = 4096
    buf, status = _buffer(1, count), torch.zeros(1, dtype=torch.int32, device="cuda")
    v = torch.randn(count, device="cuda")
    want = v.clone()
    g, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for _ in range(3):
                ext.peer_allreduce(v, [buf.data_ptr()], 0, 0, status)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(4):
        g.replay()
    torch.cuda.synchronize()
    calls = buf[: HEADER_BYTES // 4].view(torch.int32)[:CTAS]
    assert calls.tolist() == [12] * CTAS and torch.equal(v, want) and int(status.item()) == 0


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
    second) and raises the status word (nothing of that peer arrived, so nothing is written)."""
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
        ext.peer_allreduce(torch.zeros(8, device="cuda"), [buf.data_ptr()], 1, 1, status)      # rank >= world
