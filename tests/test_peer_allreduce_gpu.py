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


@pytest.mark.parametrize("spin_limit", [0, 4000])
def test_wait_runs_out_instead_of_hanging(spin_limit):
    """A peer that never delivers: the kernel gives up after its bounded wait (the default of
    about half a second, or the caller's limit), raises the status word and leaves NaN in every
    element it could not complete, so that the sums cannot be used by accident."""
    ext = _ext()
    world, count = 2, 1024
    bufs = [_buffer(world, count), _buffer(world, count)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    v = torch.randn(count, device="cuda")
    keep = v.clone()
    ext.peer_allreduce(v, [b.data_ptr() for b in bufs], 0, 1, status, spin_limit)
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert torch.isnan(v).all()
    # the context is still usable and the next collective works once the peer does deliver
    status.zero_()
    v.copy_(keep)
    _deliver(bufs[0], world, count, 0, 1, torch.ones(count, device="cuda"), 2)
    ext.peer_allreduce(v, [b.data_ptr() for b in bufs], 0, 2, status, spin_limit)
    assert int(status.item()) == 0 and torch.equal(v, keep + 1)


def test_rejects_bad_arguments():
    ext = _ext()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    buf = _buffer(1, 8)
    with pytest.raises(RuntimeError):
        ext.peer_allreduce(torch.zeros(6, device="cuda"), [buf.data_ptr()], 0, 1, status)      # count % 4
    with pytest.raises(RuntimeError):
        ext.peer_allreduce(torch.zeros(8, device="cuda"), [buf.data_ptr()], 1, 1, status)      # rank >= world


# ---- the exchange fused into the backward's finishing kernel (cc1d_bwd_params.peers) --------------
def _bwd_inputs(channel_last, B=3, D=72, L=257, W=4, dtype=torch.bfloat16):
    mk = (lambda: torch.randn(B, L, D, device="cuda", dtype=dtype).transpose(1, 2)) if channel_last else \
         (lambda: torch.randn(B, D, L, device="cuda", dtype=dtype))
    return mk(), mk(), torch.randn(D, W, device="cuda"), torch.randn(D, device="cuda")


def _bwd(x, dout, w, b, **peer):
    dx = torch.empty_like(x)
    dw, db = torch.empty_like(w), torch.empty_like(b)
    _ext().causal_conv1d_bwd(x, w, b, dout, None, None, None, dx, dw, db, None, True, False, **peer)
    return dx, dw, db


def _lines8(buf, world, capacity):
    return buf[HEADER_BYTES // 4:].view(torch.int32).view(2, world, capacity, 2)


@pytest.mark.parametrize("channel_last", [False, True])
def test_fused_exchange_world_of_one_is_the_plain_backward(channel_last):
    torch.manual_seed(3)
    x, dout, w, b = _bwd_inputs(channel_last)
    cap = w.numel() + b.numel()
    buf, status = _buffer(1, (cap + 3) // 4 * 4), torch.zeros(1, dtype=torch.int32, device="cuda")
    peer = dict(peer_ptrs=[buf.data_ptr()], peer_rank=0, peer_capacity=(cap + 3) // 4 * 4, peer_status=status)
    want = _bwd(x, dout, w, b)
    for call in range(3):                              # the epoch advances by itself
        got = _bwd(x, dout, w, b, **peer)
        assert all(torch.equal(a, c) for a, c in zip(got, want)), f"call {call}"
    stamps = _lines8(buf, 1, (cap + 3) // 4 * 4)[:, 0, :cap, 1]
    assert sorted(stamps.max(dim=1).values.tolist()) == [2, 3] and int(status.item()) == 0
    # replayable in a CUDA graph
    g, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    outs = []
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            outs = _bwd(x, dout, w, b, **peer)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert all(torch.equal(a, c) for a, c in zip(outs, want)) and int(status.item()) == 0


def test_fused_exchange_adds_what_a_peer_delivered():
    torch.manual_seed(4)
    x, dout, w, b = _bwd_inputs(False)
    D, W = w.shape
    cap = D * (W + 1)
    bufs = [_buffer(2, cap), _buffer(2, cap)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    other = torch.randn(D, W + 1, device="cuda")       # rank 1's partial: taps 0..W-1, then the bias gradient
    lines = _lines8(bufs[0], 2, cap)
    lines[1, 1, :, 0] = other.reshape(-1).view(torch.int32)   # first collective: epoch 1, parity 1
    lines[1, 1, :, 1] = 1
    _, dw0, db0 = _bwd(x, dout, w, b)
    _, dw, db = _bwd(x, dout, w, b, peer_ptrs=[bf.data_ptr() for bf in bufs], peer_rank=0, peer_capacity=cap, peer_status=status)
    assert torch.equal(dw, dw0 + other[:, :W]) and torch.equal(db, db0 + other[:, W]) and int(status.item()) == 0
    # what this rank left in the peer's buffer is its own partial, stamped 1
    sent = _lines8(bufs[1], 2, cap)[1, 0]
    assert torch.equal(sent[:, 0].view(torch.float32).view(D, W + 1)[:, :W], dw0) and (sent[:, 1] == 1).all()


def test_fused_exchange_gives_up_when_the_peer_never_delivers():
    torch.manual_seed(5)
    x, dout, w, b = _bwd_inputs(True, B=1, D=64, L=40)
    cap = w.numel() + b.numel()
    bufs = [_buffer(2, cap), _buffer(2, cap)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dx, dw, db = _bwd(x, dout, w, b, peer_ptrs=[bf.data_ptr() for bf in bufs], peer_rank=0, peer_capacity=cap,
                      peer_status=status, peer_spin_limit=4000)
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert torch.isnan(dw).all() and torch.isnan(db).all(), "sums that could not be completed must read as NaN"
    assert torch.equal(dx, _bwd(x, dout, w, b)[0]), "dx does not depend on the exchange"


@pytest.mark.parametrize("channel_last", [False, True])
def test_backward_split_into_phases_is_bit_identical(channel_last):
    """phase 1 (main kernel) and phase 2 (finishing kernel) on two streams, sharing a caller
    workspace, give the bits of the single call."""
    torch.manual_seed(6)
    ext = _ext()
    x, dout, w, b = _bwd_inputs(channel_last, B=4, D=136, L=515)
    want = _bwd(x, dout, w, b)
    ws = torch.empty(ext.bwd_workspace_bytes(x.shape[0], x.shape[1], x.shape[2], w.shape[1], x.element_size(), channel_last),
                     dtype=torch.uint8, device="cuda")
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(b)
    side = torch.cuda.Stream()
    ext.causal_conv1d_bwd(x, w, b, dout, None, None, None, dx, dw, db, None, True, False, phase=1, workspace=ws)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ext.causal_conv1d_bwd(x, w, b, dout, None, None, None, dx, dw, db, None, True, False, phase=2, workspace=ws)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    assert all(torch.equal(a, c) for a, c in zip((dx, dw, db), want))
    with pytest.raises(RuntimeError):
        ext.causal_conv1d_bwd(x, w, b, dout, None, None, None, dx, dw, db, None, True, False, phase=1)   # no workspace
