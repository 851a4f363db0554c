#!/usr/bin/env python
"""Benchmark of the causal depthwise conv1d hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (N = 1): the Mamba-1 2.8B-shape prefill, forward + backward, bf16:
x (8, 5120, 2048) channel-first, weight (5120, 4) / bias bf16, SiLU.  One step = one forward
plus one backward over one batch.  At N > 1 every rank runs the same per-GPU batch (weak
scaling) and each step ends with the single exchange of the packed fp32 dweight/dbias (one
kernel per rank over NVLink peer memory; NCCL when that cannot be set up).
The timed steps are CUDA-graph replays.  Extra keys: `kernels` (forward and backward timed
back to back), `secondary` (the packed varlen prefill, the prefill with conv states and the
decode update at N = 1; the channel-sharded decode update and the strong-scaling step at N > 1).

Prints ONE JSON line (rank 0).  `value` is whole-job algorithmic GB/s with inputs resident
in HBM; `e2e` is the same metric through the public Python API with pinned HOST buffers,
copies inside the timed region.  `--impl reference` times the CPU port of the reference's
algorithm (oracle/) on the host cores instead.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# ---- workload: Mamba-1 2.8B-shape prefill, fwd+bwd ------------------------------------------
BATCH_PER_GPU, DIM, SEQLEN, WIDTH = 8, 5120, 2048, 4
ELEM = 2  # bf16
METRIC = "fwd+bwd algorithmic HBM GB/s, Mamba-1 2.8B prefill shape (8,5120,2048) bf16 width 4 SiLU"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes of one launch of the backward kernel, from an ncu capture of this workload:
# dram__bytes_read.sum + dram__bytes_write.sum (write-back of the last ~26 MB of dx is still
# pending in L2 when the counter stops)
BWD_KERNEL_DRAM_TRAFFIC_BYTES = 335708416 + 141833984


def algorithmic_bytes(batch):
    n = batch * DIM * SEQLEN
    w = (WIDTH + 1) * DIM
    fwd = 2 * n * ELEM + w * ELEM                 # x + out, weights + bias
    bwd = 3 * n * ELEM + w * ELEM + w * 4         # x, dout, dx, weights, fp32 grads
    return fwd, bwd


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (earlier pool measurement)"


# ---- clocks ---------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (NVML,
    read-only)."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, torch_device_index, period=0.02, enabled=True):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period, self._stop, self._thread, self.ok = period, threading.Event(), None, False
        self.err = "not sampled on this rank"
        if not enabled:       # one sampler per job (rank 0): NVML polling from every rank only adds host noise
            return
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(torch_device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception as e:  # noqa: BLE001
            self.err = repr(e)

    def _read_reasons(self):
        for name in ("nvmlDeviceGetCurrentClocksEventReasons", "nvmlDeviceGetCurrentClocksThrottleReasons"):
            fn = getattr(self.nv, name, None)
            if fn is not None:
                return int(fn(self.h))
        return 0

    def _loop(self):
        while not self._stop.is_set():
            try:
                self.samples.append(int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
                bits = self._read_reasons()
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.ok:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "note": "no NVML samples"}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---- CPU port (oracle) timing -------------------------------------------------------------------
def cpu_port_inputs(batch, dim, seqlen, seed=1):
    import numpy as np
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, dim, seqlen), dtype=np.float32)
    dout = rng.standard_normal((batch, dim, seqlen), dtype=np.float32)
    w = (rng.random((dim, WIDTH), dtype=np.float32) - 0.5)
    b = (rng.random((dim,), dtype=np.float32) - 0.5)
    out, dx = np.empty_like(x), np.empty_like(x)
    dw, db = np.empty_like(w), np.empty_like(b)
    return x, dout, w, b, out, dx, dw, db


def cpu_port_step(buf):
    import oracle
    x, dout, w, b, out, dx, dw, db = buf
    t = oracle.fwd_f32_timed(x, w, b, out, WIDTH, True)
    t += oracle.bwd_f32_timed(x, w, b, dout, dx, dw, db, WIDTH, True)
    return t


def cpu_baseline(target_seconds=12.0):
    """The CPU port on a bounded sample: one batch row of the workload, repeated."""
    import oracle
    oracle.build()
    oracle.set_threads(host_cores())
    buf = cpu_port_inputs(1, DIM, SEQLEN)
    cpu_port_step(buf)  # warm-up
    n, total = 0, 0.0
    while total < target_seconds and n < 5000:
        total += cpu_port_step(buf)
        n += 1
    fwd, bwd = algorithmic_bytes(1)
    return {"value": round((fwd + bwd) * n / total / 1e9, 3), "unit": UNIT, "cores": oracle.max_threads(),
            "kind": "port", "sample": f"one batch row per step: 1 of {BATCH_PER_GPU} rows (1,{DIM},{SEQLEN}), fwd+bwd in fp32, "
                                      f"{n} repeats, {total:.1f} s; OpenMP over rows"}


def run_reference(args):
    """--impl reference: the CPU port of the reference's algorithm on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    oracle.build()
    # every host core at every N: a launcher may have exported OMP_NUM_THREADS=1 for its workers
    oracle.set_threads(host_cores())
    cores = oracle.max_threads()
    # size the per-step sample so that the whole run stays within ~2.5 minutes
    probe = cpu_port_inputs(1, 256, SEQLEN)
    cpu_port_step(probe)
    t_probe = min(cpu_port_step(probe) for _ in range(3))
    per_channel = t_probe / 256
    budget = 150.0 / max(1, args.steps + args.warmup)
    dim = int(max(64, min(DIM, budget / per_channel)))
    dim -= dim % 8
    buf = cpu_port_inputs(1, dim, SEQLEN)
    for _ in range(args.warmup):
        cpu_port_step(buf)
    total = 0.0
    for _ in range(args.steps):
        total += cpu_port_step(buf)
    n = dim * SEQLEN
    step_bytes = 5 * n * ELEM + (WIDTH + 1) * dim * (2 * ELEM + 4)
    value = step_bytes * args.steps / total / 1e9
    sample = (f"one batch row per step: a (1,{dim},{SEQLEN}) slice of the (8,{DIM},{SEQLEN}) batch, fp32 arithmetic, "
              f"fwd+bwd, OpenMP over rows on {cores} threads; CPU port of the reference's algorithm")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(total / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


ALLREDUCE_TEXT = {
    "nccl": "one NCCL all-reduce of packed fp32 dweight|dbias per step (async, overlapped with the next step's kernels; "
            "launched from the host every step)",
    "peer": "one cc1d_peer_allreduce kernel per step on the packed fp32 dweight|dbias (NVLink peer stores), on a side "
            "branch of the CUDA-graph-captured step beside the next step's kernels",
    "fused": "dweight|dbias exchanged through NVLink peer memory inside the backward's finishing kernel (one kernel does the "
             "last local reduction and the exchange), on a side branch of the CUDA-graph-captured step beside the next "
             "step's kernels",
}


def workload_config(n_gpus, allreduce="peer", graph=True):
    return {
        "workload": "C2 Mamba-1 2.8B-shape prefill fwd+bwd: x (8,5120,2048) bf16 channel-first per GPU, "
                    "weight (5120,4)+bias bf16, SiLU, dout N(0,1), seed 1",
        "batch_per_gpu": BATCH_PER_GPU, "global_batch": BATCH_PER_GPU * n_gpus, "dim": DIM, "seq_len": SEQLEN,
        "width": WIDTH, "activation": "silu",
        "parallelism": f"batch-sharded dp{n_gpus}, {ALLREDUCE_TEXT[allreduce]}" if n_gpus > 1 else "single GPU",
        "l2": "inputs larger than L2: 3 rotating buffer sets of 671 MB (x, dout, out, dx) per GPU",
        "launch": ("the K timed steps are CUDA-graph replays (graphs of up to 60 steps captured after the warm-up); in a "
                   "captured step the backward's finishing kernel runs on a side branch beside the next forward"
                   if graph else "every step launched from the host"),
        "kernel_split": "forward launches back to back, then backward launches back to back, after the timed region "
                        "(CUDA events around each loop)",
    }


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ---- the B200 arm -------------------------------------------------------------------------------
GRAPH_STEPS = 60     # steps per captured graph: a multiple of 2 (gradient buffers) and 3 (buffer sets)


def _agree(dist, torch, dev, ok):
    """True only if `ok` holds on every rank (the ranks must all take the same exchange path)."""
    t = torch.tensor([1 if ok else 0], device=dev, dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def run_b200(args):
    import torch
    import torch.distributed as dist

    from causal_conv1d_b200 import causal_conv1d_fn
    from causal_conv1d_b200._ext import ext
    from causal_conv1d_b200.distributed import packed_grad_buffer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
        args.gpus = world
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path in causal_conv1d_b200")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    B, K, Wm = BATCH_PER_GPU, args.steps, max(args.warmup, 3)
    torch.manual_seed(1 + rank)
    nsets = max(1, args.buffer_sets)
    sets = []
    for _ in range(nsets):
        x = torch.randn(B, DIM, SEQLEN, device=dev, dtype=torch.bfloat16)
        dout = torch.randn(B, DIM, SEQLEN, device=dev, dtype=torch.bfloat16)
        sets.append((x, dout, torch.empty_like(x), torch.empty_like(x)))
    gen = torch.Generator(device="cpu").manual_seed(1)
    weight = (torch.rand(DIM, WIDTH, generator=gen) - 0.5).to(device=dev, dtype=torch.bfloat16)
    bias = (torch.rand(DIM, generator=gen) - 0.5).to(device=dev, dtype=torch.bfloat16)
    # two packed gradient buffers and two scratch buffers: the exchange of step i runs beside step i+1's kernels
    grads = [packed_grad_buffer(DIM, WIDTH, True, dev) for _ in range(2)]
    ws_bytes = ext.bwd_workspace_bytes(B, DIM, SEQLEN, WIDTH, ELEM, False)
    scratch = [torch.empty(ws_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]

    # ---- which exchange (N > 1): everything is set up, and agreed on, BEFORE the warm-up steps -----------
    mode, setup_note = args.allreduce, None
    reducer = fused_reducer = aligner = None
    peer_args = {}
    if world == 1:
        mode = "single"
    else:
        if mode in ("auto", "fused", "peer"):
            ok = True
            try:
                from causal_conv1d_b200.distributed import PeerGradReducer
                n = grads[0][0].numel()
                # a wait of up to ~4 s: ranks reach their first replay at different times
                if mode in ("peer", "auto"):
                    reducer = PeerGradReducer(n, spin_limit=1 << 24)
                else:
                    fused_reducer = PeerGradReducer(n, fused=True, spin_limit=1 << 24)
                    peer_args = fused_reducer.backward_args()
                aligner = PeerGradReducer(4, spin_limit=1 << 24)    # a 16-byte all-reduce used as a device-side barrier
            except Exception as e:   # symmetric memory unavailable: every rank falls back together
                ok, setup_note = False, f"{type(e).__name__}: {e}"[:200]
            if not _agree(dist, torch, dev, ok):
                if args.allreduce != "auto":
                    raise SystemExit(f"--allreduce {args.allreduce}: peer memory could not be set up on every rank ({setup_note})")
                reducer = fused_reducer = aligner = None
                peer_args, mode = {}, "nccl"
            elif mode == "auto":
                mode = "peer"
    use_graph = mode != "nccl" and not args.no_graph
    # finishing kernel (+ exchange) on a side branch of the captured step, beside the next forward:
    # nothing in the next step depends on dweight / dbias
    split = mode in ("fused", "peer") or (mode == "single" and use_graph)
    side = torch.cuda.Stream() if split else None
    pending = [None, None]                       # NCCL work handles
    side_done = [None, None]                     # side-branch events per gradient buffer

    def step(i):
        """Enqueue step i on the current stream (and the side branch)."""
        x, dout, out, dx = sets[i % nsets]
        packed, dweight, dbias = grads[i % 2]
        main = torch.cuda.current_stream()
        if pending[i % 2] is not None:           # the buffer's previous all-reduce must be done before it is rewritten
            pending[i % 2].wait()
            pending[i % 2] = None
        if side_done[i % 2] is not None:         # ... and so must its previous finishing kernel / exchange
            main.wait_event(side_done[i % 2])
            side_done[i % 2] = None
        ext.causal_conv1d_fwd(x, weight, bias, None, None, out, None, True)
        if split:
            ext.causal_conv1d_bwd(x, weight, bias, dout, None, None, None, dx, dweight, dbias, None, True, False,
                                  phase=1, workspace=scratch[i % 2])
            ready = torch.cuda.Event()
            ready.record(main)
            side.wait_event(ready)
            with torch.cuda.stream(side):
                ext.causal_conv1d_bwd(x, weight, bias, dout, None, None, None, dx, dweight, dbias, None, True, False,
                                      phase=2, workspace=scratch[i % 2], **peer_args)
                if reducer is not None:
                    reducer.reduce_(packed)
                side_done[i % 2] = torch.cuda.Event()
                side_done[i % 2].record(side)
        else:
            ext.causal_conv1d_bwd(x, weight, bias, dout, None, None, None, dx, dweight, dbias, None, True, False)
            if mode == "nccl":
                pending[i % 2] = dist.all_reduce(packed, async_op=True)

    def drain():
        main = torch.cuda.current_stream()
        for j in range(2):
            if side_done[j] is not None:
                main.wait_event(side_done[j])
                side_done[j] = None
            if pending[j] is not None:
                pending[j].wait()
                pending[j] = None

    def barrier():
        drain()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up: W eager steps (lazy loading, communicator, peer mappings), then the graphs ---------------
    barrier()
    for i in range(Wm):
        step(i)
    barrier()
    graphs = []                                  # (graph, steps in it), in replay order for the K timed steps
    if use_graph:
        cap = torch.cuda.Stream()
        cap.wait_stream(torch.cuda.current_stream())
        made = {}
        plan = [GRAPH_STEPS] * (K // GRAPH_STEPS) + ([K % GRAPH_STEPS] if K % GRAPH_STEPS else [])
        for n in sorted(set(plan)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(cap):
                with torch.cuda.graph(g, stream=cap):
                    for i in range(n):               # every graph starts at a step index that is 0 mod 6
                        step(i)
                    drain()                          # join the side branch before the capture ends
            made[n] = g
        torch.cuda.current_stream().wait_stream(cap)
        graphs = [(made[n], n) for n in plan]
        barrier()
        for g, _ in graphs[-1:]:                     # one untimed replay: graph upload, first-launch cost
            g.replay()
        barrier()

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tiny = torch.zeros(4, device=dev)
    with ClockSampler(local_rank, period=0.002, enabled=rank == 0) as clocks:
        if aligner is not None:
            aligner.reduce_(tiny)                # device-side barrier: the GPUs start within microseconds of each other
        start.record()
        if use_graph:
            for g, _ in graphs:
                g.replay()
        else:
            for i in range(K):
                step(i)
            drain()                              # every exchange completes inside the timed region
        end.record()
        barrier()
    total_ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    for r in (reducer, fused_reducer, aligner):
        if r is not None:
            r.check()                            # a bounded wait that ran out would have left NaN sums
    ms_per_step = total_ms / K
    fwd_b, bwd_b = algorithmic_bytes(B)
    value = (fwd_b + bwd_b) * world / (ms_per_step * 1e-3) / 1e9

    # ---- per-kernel durations: each kernel launched back to back, outside the timed region ----------------
    def loop_ms(fn, n):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    n_split = min(max(K, 100), 1000)
    dw_l, db_l = torch.empty(DIM, WIDTH, device=dev), torch.empty(DIM, device=dev)
    with ClockSampler(local_rank, period=0.002, enabled=rank == 0) as clocks_split:
        fwd_ms = loop_ms(lambda i: ext.causal_conv1d_fwd(sets[i % nsets][0], weight, bias, None, None, sets[i % nsets][2],
                                                         None, True), n_split)
        bwd_ms = loop_ms(lambda i: ext.causal_conv1d_bwd(sets[i % nsets][0], weight, bias, sets[i % nsets][1], None, None, None,
                                                         sets[i % nsets][3], dw_l, db_l, None, True, False), n_split)
        # the dominant kernel alone (phase 1: dx and the partial rows; the finishing kernel not launched)
        bwd_main_ms = loop_ms(lambda i: ext.causal_conv1d_bwd(sets[i % nsets][0], weight, bias, sets[i % nsets][1], None, None,
                                                              None, sets[i % nsets][3], dw_l, db_l, None, True, False,
                                                              phase=1, workspace=scratch[0]), n_split)
    barrier()

    if args.skip_e2e:
        if rank == 0:
            print(json.dumps({"partial": True, "ms_per_step": ms_per_step, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "bwd_main_ms": bwd_main_ms,
                              "value": value, "mode": mode, "graph": use_graph}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end: public API, pinned host buffers, copies inside the timed region -------------
    k_e2e = max(3, min(K, 200))      # the pipeline's fill and drain (one copy each way without its partner) are inside
    hx = torch.randn(B, DIM, SEQLEN, dtype=torch.bfloat16).pin_memory()
    hdout = torch.randn(B, DIM, SEQLEN, dtype=torch.bfloat16).pin_memory()
    hout, hdx = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()
    hdw = torch.empty(DIM, WIDTH, dtype=torch.bfloat16).pin_memory()
    hdb = torch.empty(DIM, dtype=torch.bfloat16).pin_memory()
    # Three streams, the way a host-fed pipeline is normally written: step i's host->device copies,
    # step i-1's kernels and step i-2's device->host copies overlap (PCIe is full duplex).  Every
    # step still pays for all of its own copies inside the timed region.
    # With n copy streams every large tensor travels as n batch slices on n streams per direction.  Which n
    # keeps more of the host link busy differs from host to host (measured: 1 stream 116 GB/s against 111 GB/s
    # with 2 on one box, 92 against 107-110 on another), so --e2e-copy-streams 0 (the default) tries 1 and 2 for
    # a few steps outside the timed region and takes the faster.
    s_run = torch.cuda.Stream()
    dev_slots = [(torch.empty(B, DIM, SEQLEN, device=dev, dtype=torch.bfloat16),
                  torch.empty(B, DIM, SEQLEN, device=dev, dtype=torch.bfloat16)) for _ in range(2)]
    wps = [weight.clone().requires_grad_() for _ in range(2)]
    bps = [bias.clone().requires_grad_() for _ in range(2)]

    def run_e2e(ncs, steps, warm=2):
        cuts = [(k * B // ncs, (k + 1) * B // ncs) for k in range(ncs)]
        s_ins, s_outs = [torch.cuda.Stream() for _ in range(ncs)], [torch.cuda.Stream() for _ in range(ncs)]
        slots = [{"x": dev_slots[k][0], "dout": dev_slots[k][1],
                  "in_done": [torch.cuda.Event() for _ in range(ncs)], "run_done": torch.cuda.Event(),
                  "out_done": [torch.cuda.Event() for _ in range(ncs)]} for k in range(2)]

        def e2e_step(i):
            sl, wq, bq = slots[i % 2], wps[i % 2], bps[i % 2]
            for j, (lo, hi) in enumerate(cuts):
                st = s_ins[j]
                with torch.cuda.stream(st):
                    st.wait_event(sl["run_done"])        # the slot's previous kernels have read x / dout
                    sl["x"][lo:hi].copy_(hx[lo:hi], non_blocking=True)
                    sl["dout"][lo:hi].copy_(hdout[lo:hi], non_blocking=True)
                    sl["in_done"][j].record(st)
            with torch.cuda.stream(s_run):
                for j in range(ncs):
                    s_run.wait_event(sl["in_done"][j])
                    s_run.wait_event(sl["out_done"][j])  # the slot's previous results have left the device
                xd = sl["x"].detach().requires_grad_()
                wq.grad = bq.grad = None
                out = causal_conv1d_fn(xd, wq, bq, activation="silu")
                out.backward(sl["dout"])
                if world > 1:
                    dist.all_reduce(wq.grad)
                    dist.all_reduce(bq.grad)
                sl["run_done"].record()
            od, dxg = out.detach(), xd.grad
            for j, (lo, hi) in enumerate(cuts):
                st = s_outs[j]
                with torch.cuda.stream(st):
                    st.wait_event(sl["run_done"])
                    for t in (od, dxg, wq.grad, bq.grad):
                        t.record_stream(st)
                    hout[lo:hi].copy_(od[lo:hi], non_blocking=True)
                    hdx[lo:hi].copy_(dxg[lo:hi], non_blocking=True)
                    if j == 0:
                        hdw.copy_(wq.grad, non_blocking=True)
                        hdb.copy_(bq.grad, non_blocking=True)
                    sl["out_done"][j].record(st)

        all_streams = [s_run] + s_ins + s_outs

        def e2e_join():
            cur = torch.cuda.current_stream()
            for st in all_streams:
                cur.wait_stream(st)

        for st in all_streams:
            st.wait_stream(torch.cuda.current_stream())
        for i in range(warm):
            e2e_step(i)
        e2e_join()
        barrier()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        for st in all_streams:
            st.wait_event(s2)
        for i in range(steps):
            e2e_step(i)
        e2e_join()
        e2.record()
        barrier()
        ms = s2.elapsed_time(e2)
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    if args.e2e_copy_streams > 0:
        ncs = max(1, min(B, args.e2e_copy_streams))
    else:
        trial = {n: run_e2e(n, 4) for n in (1, 2) if n <= B}     # max over ranks: every rank picks the same n
        ncs = min(trial, key=trial.get)
    e2e_ms = run_e2e(ncs, k_e2e)
    e2e_value = (fwd_b + bwd_b) * world / (e2e_ms / k_e2e * 1e-3) / 1e9
    h2d = hx.numel() * ELEM + hdout.numel() * ELEM
    d2h = hout.numel() * ELEM + hdx.numel() * ELEM + hdw.numel() * ELEM + hdb.numel() * ELEM
    del hx, hdout, hout, hdx, dev_slots

    # ---- the exchange step alone: NCCL all-reduce vs the one-shot peer-memory kernel --------------
    allreduce_us = None
    if world > 1 and args.measure_allreduce:
        allreduce_us = {"bytes": grads[0][0].numel() * 4, "mode_of_the_timed_steps": mode}
        probe = torch.randn(grads[0][0].numel(), device=dev)

        def timed(fn, n=200):
            for _ in range(10):
                fn()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / n * 1e3], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return round(float(t.item()), 2)

        allreduce_us["nccl"] = timed(lambda: dist.all_reduce(probe))
        try:
            from causal_conv1d_b200.distributed import PeerGradReducer
            red = reducer if reducer is not None else PeerGradReducer(probe.numel(), spin_limit=1 << 24)
            allreduce_us["peer_memory_kernel"] = timed(lambda: red.reduce_(probe))
            red.check()
        except Exception as e:   # symmetric memory unavailable on this box: report, keep the bench line
            allreduce_us["peer_memory_kernel"] = None
            allreduce_us["peer_memory_kernel_error"] = f"{type(e).__name__}: {e}"[:200]

    # ---- the other workloads the configuration names, as extra keys ---------------------------------------
    secondary = None
    if not args.no_secondary:
        torch.cuda.empty_cache()
        try:
            if world == 1:
                secondary = secondary_single_gpu(torch, ext, dev)
            else:
                secondary = secondary_multi_gpu(torch, dist, ext, dev, rank, world, aligner)
        except Exception as e:   # never lose the headline line to a secondary workload
            secondary = {"error": f"{type(e).__name__}: {e}"[:300]}

    if rank == 0:
        peak, peak_src = measured_peak()
        bwd_gbs = bwd_b / (bwd_ms * 1e-3) / 1e9
        fwd_gbs = fwd_b / (fwd_ms * 1e-3) / 1e9
        main_b = bwd_b - (WIDTH + 1) * DIM * 4          # the fp32 gradients are written by the finishing kernel
        main_gbs = main_b / (bwd_main_ms * 1e-3) / 1e9
        launches_per_step = 3 + (1 if mode == "peer" else 0)
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world, mode if world > 1 else "peer", use_graph),
            "clocks": clocks.summary(),
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": k_e2e, "api": "causal_conv1d_fn + autograd backward, pinned host tensors; copy-in / kernels / copy-out of "
                           f"consecutive steps overlap ({ncs} copy stream(s) per direction)"},
            "gpu_launches": launches_per_step * K,
            "roofline": {"bound": "hbm", "kernel": "bwd_cf_wide_kernel (launched alone: cc1d_bwd phase 1)",
                         "achieved": round(main_gbs, 1), "peak": peak, "unit": UNIT, "frac": round(main_gbs / peak, 4),
                         "traffic": BWD_KERNEL_DRAM_TRAFFIC_BYTES, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": main_b, "avg_launch_ms": round(bwd_main_ms, 5),
                         "launches_timed": n_split, "frac_of_nominal_8TBs": round(main_gbs / NOMINAL_HBM_GBS, 4),
                         "with_finishing_kernel": {"achieved": round(bwd_gbs, 1), "frac": round(bwd_gbs / peak, 4),
                                                   "avg_launch_pair_ms": round(bwd_ms, 5)}},
            "kernels": {"fwd_cf_wide_kernel": {"gbs": round(fwd_gbs, 1), "ms": round(fwd_ms, 5), "frac": round(fwd_gbs / peak, 4)},
                        "bwd_cf_wide_kernel": {"gbs": round(main_gbs, 1), "ms": round(bwd_main_ms, 5), "frac": round(main_gbs / peak, 4)},
                        "bwd_cf_wide_kernel + reduce_partials_kernel": {"gbs": round(bwd_gbs, 1), "ms": round(bwd_ms, 5),
                                                                       "frac": round(bwd_gbs / peak, 4)},
                        "step": {"gbs": round(value / world, 1), "ms": round(ms_per_step, 5), "frac": round(value / world / peak, 4)},
                        "launches_timed": n_split, "clocks": clocks_split.summary()},
            "tokens_per_s": round(B * world * SEQLEN / (ms_per_step * 1e-3), 1),
        }
        if setup_note is not None:
            line["exchange_setup_note"] = setup_note
        if allreduce_us is not None:
            line["allreduce_us"] = allreduce_us
        if secondary is not None:
            line["secondary"] = secondary
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ---- secondary workloads (same JSON shape; the default stays the C2 line above) ---------------------
def _time_steps(torch, fn, nsets, steps, warmup):
    for i in range(max(warmup, 3)):
        fn(i % nsets)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(steps):
        fn(i % nsets)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / steps   # ms


def _c3_pack(torch, L, nseq=16):
    """16 sequence lengths drawn from U[256, 3840] and rescaled to sum to L (seed set by the caller)."""
    lens = torch.randint(256, 3841, (nseq,)).double()
    lens = (lens / lens.sum() * L).long()
    lens[-1] = L - lens[:-1].sum()
    return lens


def measure_c3(torch, ext, dev, steps, warmup, nsets):
    """Packed varlen prefill, channel-last, seq_idx (Mamba-2 2.7B shape), forward and backward."""
    peak, peak_src = measured_peak()
    bf = torch.bfloat16
    D, L, W = 5376, 32768, 4
    torch.manual_seed(2)
    lens = _c3_pack(torch, L)
    sidx = torch.repeat_interleave(torch.arange(16), lens).int().view(1, L).to(dev)
    w = (torch.rand(D, W) - 0.5).to(dev, bf)
    b = (torch.rand(D) - 0.5).to(dev, bf)
    sets = []
    for _ in range(nsets):
        x = torch.randn(1, L, D, device=dev, dtype=bf).transpose(1, 2)
        dout = torch.randn(1, L, D, device=dev, dtype=bf).transpose(1, 2)
        sets.append((x, dout, torch.empty_like(x), torch.empty_like(x)))
    dw, db = torch.empty(D, W, device=dev), torch.empty(D, device=dev)
    fwd = lambda i: ext.causal_conv1d_fwd(sets[i][0], w, b, sidx, None, sets[i][2], None, True)
    bwd = lambda i: ext.causal_conv1d_bwd(sets[i][0], w, b, sets[i][1], sidx, None, None, sets[i][3], dw, db, None, True, False)
    t_f = _time_steps(torch, fwd, nsets, steps, warmup)
    t_b = _time_steps(torch, bwd, nsets, steps, warmup)
    n = D * L
    fb, bb = 2 * n * ELEM + 4 * L, 3 * n * ELEM + 4 * L
    return {"metric": "fwd+bwd algorithmic HBM GB/s, Mamba-2 2.7B packed varlen prefill (1,5376,32768) bf16 channel-last, seq_idx",
            "value": round((fb + bb) / ((t_f + t_b) * 1e-3) / 1e9, 1), "unit": UNIT, "n_gpus": 1, "steps": steps,
            "warmup": max(warmup, 3), "ms_per_step": round(t_f + t_b, 5), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": "C3a packed varlen prefill: 16 sequences, 32768 tokens, dim 5376, width 4, SiLU, seed 2",
                                            "l2": f"{nsets} rotating buffer sets of 1.4 GB"},
            "kernels": {"fwd_cl (TMA)": {"ms": round(t_f, 5), "gbs": round(fb / t_f / 1e6, 1), "frac": round(fb / t_f / 1e6 / peak, 4)},
                        "bwd_cl (TMA) + reduce": {"ms": round(t_b, 5), "gbs": round(bb / t_b / 1e6, 1), "frac": round(bb / t_b / 1e6 / peak, 4)}},
            "roofline": {"bound": "hbm", "kernel": "bwd_cl_tma_kernel (+ reduce_partials_kernel)", "achieved": round(bb / t_b / 1e6, 1),
                         "peak": peak, "unit": UNIT, "frac": round(bb / t_b / 1e6 / peak, 4), "traffic": None, "peak_source": peak_src},
            "gpu_launches": 3 * steps, "tokens_per_s": round(L / ((t_f + t_b) * 1e-3), 1)}


def measure_c3p(torch, ext, dev, steps, warmup, nsets):
    """The C3 pack as a serving prefill: every sequence continues from, and leaves behind, a row of a
    conv-state pool (one cc1d_prefill_varlen call = masked forward + boundary kernel)."""
    peak, peak_src = measured_peak()
    bf = torch.bfloat16
    D, L, W, S, NSEQ, POOL = 5376, 32768, 4, 3, 16, 64
    torch.manual_seed(2)
    lens = _c3_pack(torch, L, NSEQ)
    cu = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).int().to(dev)
    sidx = torch.empty(L, dtype=torch.int32, device=dev)
    ext.seq_idx_from_cu_seqlens(cu, sidx)
    w = (torch.rand(D, W) - 0.5).to(dev, bf)
    b = (torch.rand(D) - 0.5).to(dev, bf)
    rows = torch.randperm(POOL)[:NSEQ].int().to(dev)
    pool = torch.randn(POOL, S, D, device=dev, dtype=bf).transpose(1, 2)
    sets = []
    for _ in range(nsets):
        x = torch.randn(L, D, device=dev, dtype=bf)
        sets.append((x, torch.empty_like(x)))
    states_out = torch.empty(NSEQ, S, D, device=dev, dtype=bf).transpose(1, 2)
    fused = lambda i: ext.causal_conv1d_prefill_varlen(sets[i][0], w, b, sidx, cu, pool, pool, rows, None, sets[i][1], True)
    plain = lambda i: ext.causal_conv1d_fwd(sets[i][0].T.unsqueeze(0), w, b, sidx.view(1, L), None,
                                            sets[i][1].T.unsqueeze(0), None, True)
    two_pass = lambda i: (plain(i), ext.causal_conv1d_varlen_states(sets[i][0], cu, states_out))
    t_fused = _time_steps(torch, fused, nsets, steps, warmup)
    t_plain = _time_steps(torch, plain, nsets, steps, warmup)
    t_two = _time_steps(torch, two_pass, nsets, steps, warmup)
    byts = 2 * D * L * ELEM + 4 * L + 2 * NSEQ * D * S * ELEM
    return {"metric": "packed varlen prefill with per-sequence conv states, algorithmic HBM GB/s, (32768 tokens, dim 5376) bf16",
            "value": round(byts / t_fused / 1e6, 1), "unit": UNIT, "n_gpus": 1, "steps": steps,
            "warmup": max(warmup, 3), "ms_per_step": round(t_fused, 5), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "C3 pack (16 sequences, 32768 tokens, dim 5376, width 4, SiLU, seed 2), each sequence prefixed by "
                                   "and written back to its row of a (64, 5376, 3) state pool",
                       "l2": f"{nsets} rotating x/out sets of 705 MB"},
            "calls": {"cc1d_prefill_varlen (masked forward + boundary kernel)": {"ms": round(t_fused, 5)},
                      "masked forward alone (no states)": {"ms": round(t_plain, 5)},
                      "masked forward + cc1d_varlen_states (two calls, no prefix possible)": {"ms": round(t_two, 5)}},
            "roofline": {"bound": "hbm", "kernel": "fwd_cl_tma_kernel (+ prefill_boundary_kernel)", "achieved": round(byts / t_fused / 1e6, 1),
                         "peak": peak, "unit": UNIT, "frac": round(byts / t_fused / 1e6 / peak, 4), "traffic": None,
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": byts},
            "gpu_launches": 2 * steps, "tokens_per_s": round(L / (t_fused * 1e-3), 1)}


def c4_algorithmic_bytes(B, D, W, Lx, S, circular):
    per = (2 * Lx + (W - 1) + Lx) if circular else (2 * Lx + max(W - 1, S - Lx) + S)
    return B * D * ELEM * per + 4 * B * (2 if circular else 1)


def time_decode_variant(torch, ext, dev, B, D, W, POOL, idx, w, b, cl, Lx, S, circ, steps, warmup, nsets, public_api=False):
    """One decode-update variant: back-to-back launches, CUDA-graph replay, and (optionally) the public
    causal_conv1d_update call, which allocates its output."""
    bf = torch.bfloat16
    sets = []
    for _ in range(nsets):
        x = torch.randn(B, Lx, D, device=dev, dtype=bf).transpose(1, 2) if (cl and Lx > 1) else torch.randn(B, D, Lx, device=dev, dtype=bf)
        st = torch.randn(POOL, S, D, device=dev, dtype=bf).transpose(1, 2) if cl else torch.randn(POOL, D, S, device=dev, dtype=bf)
        sets.append((x, st, torch.empty_like(x)))
    cache = torch.randint(0, 10000, (B,), dtype=torch.int32, device=dev) if circ else None
    run = lambda i: ext.causal_conv1d_update(sets[i][0], sets[i][1], w, b, sets[i][2], True, cache, idx)
    t_stream = _time_steps(torch, run, nsets, steps, warmup)
    g, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(nsets):
            run(i)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=side):
            for i in range(nsets):
                run(i)
    t_graph = _time_steps(torch, lambda i: g.replay(), 1, max(3, steps // nsets), 3) / nsets
    r = {"us_stream": round(t_stream * 1e3, 3), "us_graph": round(t_graph * 1e3, 3)}
    if public_api:
        from causal_conv1d_b200 import causal_conv1d_update
        xs = [s_[0].squeeze(-1) if Lx == 1 else s_[0] for s_ in sets]
        pub = lambda i: causal_conv1d_update(xs[i], sets[i][1], w, b, activation="silu", cache_seqlens=cache,
                                             conv_state_indices=idx)
        r["us_public_api"] = round(_time_steps(torch, pub, nsets, steps, warmup) * 1e3, 3)
    return r


def measure_c4(torch, ext, dev, steps, warmup, nsets, D=5376, label="C4 decode update, seqlen 1, SiLU, seed 3"):
    """Decode update, batch 256, pool of 512 states gathered by conv_state_indices: us per step for
    both state layouts and for the variants (4 tokens, circular pool of 8 slots, both)."""
    peak, peak_src = measured_peak()
    bf = torch.bfloat16
    B, S, W, POOL = 256, 3, 4, 512
    torch.manual_seed(3)
    nsets = max(nsets, 8)   # 8 x 22 MB > L2
    w = (torch.rand(D, W) - 0.5).to(dev, bf)
    b = (torch.rand(D) - 0.5).to(dev, bf)
    idx = torch.randperm(POOL)[:B].int().to(dev)
    args_ = (torch, ext, dev, B, D, W, POOL, idx, w, b)
    res, variants = {}, {}
    for name, cl in (("channel_last_state", True), ("contiguous_state", False)):
        r = time_decode_variant(*args_, cl, 1, S, False, steps, warmup, nsets, public_api=True)
        r["algorithmic_bytes"] = c4_algorithmic_bytes(B, D, W, 1, S, False)
        r["lower_bound_us"] = round(r["algorithmic_bytes"] / peak / 1e3, 3)
        r["x_bound"] = round(r["us_graph"] / r["lower_bound_us"], 2)
        res[name] = r
    for name, cl in (("channel_last_state", True), ("contiguous_state", False)):
        for Lx, S_, circ in ((4, 3, False), (1, 8, True), (4, 8, True)):
            r = time_decode_variant(*args_, cl, Lx, S_, circ, steps, warmup, nsets)
            r["algorithmic_bytes"] = c4_algorithmic_bytes(B, D, W, Lx, S_, circ)
            r["lower_bound_us"] = round(r["algorithmic_bytes"] / peak / 1e3, 3)
            r["x_bound"] = round(r["us_graph"] / r["lower_bound_us"], 2)
            if circ and not cl:
                # rows of 16 bytes: every 32-byte sector of a touched state block is read and written back whole
                r["sector_bytes"] = B * D * ELEM * (2 * Lx + 2 * S_)
            variants[f"{name}, seqlen {Lx}, state_len {S_}, {'circular' if circ else 'linear'}"] = r
    byts = c4_algorithmic_bytes(B, D, W, 1, S, False)
    best = min(r["us_graph"] for r in res.values())
    return {"metric": f"decode update us per step, batch 256, dim {D}, bf16, pool of 512 states (state_len 3), gathered by conv_state_indices",
            "value": best, "unit": "us", "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3),
            "ms_per_step": round(best * 1e-3, 6), "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": label, "l2": f"{nsets} rotating x/state/out sets (> 2x L2)",
                       "timing": "us_stream: back-to-back launches; us_graph: CUDA-graph replay of the same launches; "
                                 "us_public_api: causal_conv1d_update as a user calls it (allocates the output)"},
            "layouts": res, "variants": variants,
            "roofline": {"bound": "hbm", "kernel": "update_vec_kernel / update_cfstate_kernel", "achieved": round(byts / best / 1e3, 1),
                         "peak": peak, "unit": UNIT, "frac": round(byts / best / 1e3 / peak, 4), "traffic": None,
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": byts,
                         "lower_bound_us": round(byts / peak / 1e3, 3)},
            "gpu_launches": steps}


def secondary_single_gpu(torch, ext, dev):
    """The other single-GPU workloads of the configuration list, compacted into one object."""
    out = {}
    c3 = measure_c3(torch, ext, dev, 60, 5, 3)
    out["c3a_packed_varlen_channel_last_seq_idx"] = {"ms_fwd_bwd": c3["ms_per_step"], "gbs": c3["value"],
                                                     "kernels": c3["kernels"], "tokens_per_s": c3["tokens_per_s"]}
    torch.cuda.empty_cache()
    c3p = measure_c3p(torch, ext, dev, 60, 5, 3)
    out["c3p_prefill_with_conv_states"] = {"ms": c3p["ms_per_step"], "gbs": c3p["value"], "frac": c3p["roofline"]["frac"],
                                           "calls": c3p["calls"]}
    torch.cuda.empty_cache()
    c4 = measure_c4(torch, ext, dev, 400, 10, 8)
    out["c4_decode_update"] = {"us_per_step": c4["value"], "layouts": c4["layouts"], "variants": c4["variants"],
                               "timing": c4["config"]["timing"]}
    return out


def secondary_multi_gpu(torch, dist, ext, dev, rank, world, aligner):
    """N > 1: the decode update channel-sharded (dim 5376 / N per GPU, no communication) and the C2
    step under strong scaling (global batch 8, 8 / N rows per GPU, exchange fused into the finishing
    kernel, CUDA graph).  Times are the max over ranks."""
    from causal_conv1d_b200.distributed import PeerGradReducer, packed_grad_buffer

    def max_over_ranks(v):
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {}
    # ---- decode update, channel shard ----
    bf = torch.bfloat16
    D = 5376 // 8 // world * 8
    B, W, POOL, S = 256, 4, 512, 3
    torch.manual_seed(3)
    w = (torch.rand(D, W) - 0.5).to(dev, bf)
    b = (torch.rand(D) - 0.5).to(dev, bf)
    idx = torch.randperm(POOL)[:B].int().to(dev)
    nsets = 8 * world      # the shard is 22 MB / N: keep the rotation larger than L2
    r = time_decode_variant(torch, ext, dev, B, D, W, POOL, idx, w, b, True, 1, S, False, 400, 10, nsets)
    out["c4_decode_update_channel_sharded"] = {
        "dim_per_gpu": D, "us_graph": round(max_over_ranks(r["us_graph"]), 3), "us_stream": round(max_over_ranks(r["us_stream"]), 3),
        "algorithmic_bytes_per_gpu": c4_algorithmic_bytes(B, D, W, 1, S, False), "collective": "none"}
    torch.cuda.empty_cache()
    # ---- C2, strong scaling ----
    if BATCH_PER_GPU % world == 0:
        Bl = BATCH_PER_GPU // world
        nsets = 3 * world
        sets = []
        for _ in range(nsets):
            x = torch.randn(Bl, DIM, SEQLEN, device=dev, dtype=bf)
            dout = torch.randn(Bl, DIM, SEQLEN, device=dev, dtype=bf)
            sets.append((x, dout, torch.empty_like(x), torch.empty_like(x)))
        w2 = (torch.rand(DIM, WIDTH) - 0.5).to(dev, bf)
        b2 = (torch.rand(DIM) - 0.5).to(dev, bf)
        grads = [packed_grad_buffer(DIM, WIDTH, True, dev) for _ in range(2)]
        red = PeerGradReducer(grads[0][0].numel(), fused=True, spin_limit=1 << 24)
        pa = red.backward_args()

        def one(i):
            x, dout, o, dx = sets[i % nsets]
            _, dwt, dbs = grads[i % 2]
            ext.causal_conv1d_fwd(x, w2, b2, None, None, o, None, True)
            ext.causal_conv1d_bwd(x, w2, b2, dout, None, None, None, dx, dwt, dbs, None, True, False, **pa)

        for i in range(4):
            one(i)
        dist.barrier()
        torch.cuda.synchronize()
        n_cap = 2 * nsets
        g, cap = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        cap.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cap):
            with torch.cuda.graph(g, stream=cap):
                for i in range(n_cap):
                    one(i)
        torch.cuda.current_stream().wait_stream(cap)
        dist.barrier()
        torch.cuda.synchronize()
        g.replay()
        dist.barrier()
        torch.cuda.synchronize()
        reps = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if aligner is not None:
            aligner.reduce_(torch.zeros(4, device=dev))
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1) / (reps * n_cap))
        red.check()
        fwd_b, bwd_b = algorithmic_bytes(BATCH_PER_GPU)
        out["c2_strong_scaling"] = {"global_batch": BATCH_PER_GPU, "rows_per_gpu": Bl, "ms_per_step": round(ms, 5),
                                    "gbs": round((fwd_b + bwd_b) / (ms * 1e-3) / 1e9, 1), "steps": reps * n_cap,
                                    "exchange": "fused into the finishing kernel, in stream, CUDA graph"}
    return out


def run_secondary(args):
    """--workload c3: packed varlen prefill, channel-last, seq_idx, fwd+bwd.
    --workload c3p: the same pack through cc1d_prefill_varlen (forward with per-sequence conv states).
    --workload c4: decode update, batch 256, pool of 512 states, us per step."""
    import torch

    from causal_conv1d_b200._ext import ext

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    nsets = max(1, args.buffer_sets)
    fn = {"c3": measure_c3, "c3p": measure_c3p, "c4": measure_c4}[args.workload]
    print(json.dumps(fn(torch, ext, dev, args.steps, args.warmup, nsets)), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the ~12 s CPU-port timing")
    ap.add_argument("--buffer-sets", type=int, default=3, help="rotating input/output sets (profiling: 1)")
    ap.add_argument("--skip-e2e", action="store_true", help="kernel loop only (for ncu captures)")
    ap.add_argument("--allreduce", default="auto", choices=["auto", "nccl", "peer", "fused"],
                    help="N > 1: auto (default) = peer when peer memory can be set up on every rank, else nccl; peer: the "
                         "one-shot peer-memory all-reduce kernel after the backward; fused: the exchange inside the "
                         "backward's finishing kernel; nccl: NCCL all-reduce launched from the host")
    ap.add_argument("--e2e-copy-streams", type=int, default=0,
                    help="streams (batch slices in flight) per direction in the end-to-end measurement; 0: try 1 and 2, take the faster")
    ap.add_argument("--no-graph", action="store_true", help="launch every timed step from the host instead of replaying CUDA graphs")
    ap.add_argument("--no-secondary", action="store_true", help="skip the extra workloads reported under `secondary`")
    ap.add_argument("--measure-allreduce", action="store_true",
                    help="N > 1: also time the exchange step alone, NCCL against the peer-memory kernel (sets up symmetric memory)")
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c3p", "c4"],
                    help="c2 (default, the headline line); c3: packed varlen channel-last prefill fwd+bwd; "
                         "c3p: the same pack as a serving prefill with per-sequence conv states; c4: decode update")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "c2":
        run_secondary(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
