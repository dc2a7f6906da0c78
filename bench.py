#!/usr/bin/env python
"""Benchmark of the segment-memory hot path: tokens/s of the chunked linear-memory update + query on
the kernel-alone configuration (B=8, H=8, T=2048, d_k=d_v=64, bf16 inputs, fp32 carried state), one
such batch per launch, weak scaling over GPUs (every rank runs its own batches, no collective on the
data path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl engine|reference]

N > 1 is launched by ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``; rank 0
prints ONE JSON line.

A step is ``--batches-per-step`` (default 128) consecutive batches, each one launch of the scan kernel
over inputs that rotate through more buffers than L2 holds; the batches of a step are one CUDA graph and
the timed region is K replays of it between one pair of CUDA events (W replays before it untimed), so at
the default K the region lasts tens of milliseconds and the clock sampler sees it.

Keys beyond the base contract:

* ``roofline``      -- the scan kernel against the HBM roofline (algorithmic bytes per launch / mean
                       launch time from the events above), the tensor-pipe figures beside it;
* ``cpu_baseline``  -- the reference's default CPU path (``grm.core.cuda_ops.cuda_chunk_update`` on CPU
                       tensors, i.e. its vectorised PyTorch math driven per 64- or 128-token call) timed on
                       this host's cores, its compiled sequential C++ op beside it;
* ``e2e``           -- the same metric through ``cuda_ops.cuda_chunk_update`` from pinned host buffers:
                       one host->device copy of the packed inputs and one device->host copy of the packed
                       results per batch, inside the timed region;
* ``scale_out``     -- configuration 5 (4096 rows x 32768 tokens, d=128, segment 1024, top-k 8) with its
                       rows sharded over the N GPUs (strong scaling), sample rows gathered over NCCL and
                       checked against the oracle;
* ``other_workloads`` -- retrieval (config 3), the config-4 model, backward, N=1 only.

``--impl reference`` times the reference's CPU code on the same workload (same ``config.workload``,
same steps, one batch per step); it and ``cpu_baseline`` are the only legs that execute ``oracle/``.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

CFG2 = dict(B=8, Hd=8, T=2048, K=64, V=64, decay=0.97)
CFG3 = dict(B=16, Hd=8, T=8192, segment=256, K=64, V=64, top_k=4)
CFG4 = dict(B=8, T=8192, layers=4, hidden=512, K=64, segment=512, top_k=4, vocab=32768, decay=0.97)
L2_BYTES = 126 * 1024 * 1024
WORKLOAD = ("chunked linear-memory update + query kernel alone: B=8 H=8 T=2048 d_k=64 d_v=64, decay 0.97, "
            "zero start state")
PROFILE_FIGURES = ROOT / "profiles" / "ncu_figures.json"


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), float(data["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def profile_figure(*keys):
    """A figure copied from an ncu capture, kept beside the summary it came from (profiles/); None when
    the file or the entry is missing."""
    try:
        node = json.loads(PROFILE_FIGURES.read_text())
        for key in keys:
            node = node[key]
        return node
    except (OSError, KeyError, ValueError, TypeError):
        return None


def bind_to_gpu_numa_node(device_index: int):
    """Pin this process to the cores of the NUMA node its GPU hangs off, before any pinned host memory is
    allocated (first touch then places the buffers on that node).  Returns a description, or why not."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        bus = pynvml.nvmlDeviceGetPciInfo(handle).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        bus = bus.lower()
        if len(bus.split(":")[0]) == 8:                 # NVML pads the domain to 8 digits, sysfs uses 4
            bus = bus[4:]
        node = int((Path("/sys/bus/pci/devices") / bus / "numa_node").read_text())
        if node < 0:
            return "no NUMA information for the GPU"
        cpus = set()
        for part in (Path("/sys/devices/system/node") / f"node{node}" / "cpulist").read_text().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return f"node {node} has no core this process may use"
        os.sched_setaffinity(0, allowed)
        return f"node {node}, {len(allowed)} cores"
    except Exception as exc:                              # no NVML, no sysfs entry, not Linux ...
        return f"not bound ({type(exc).__name__})"


class ClockSampler:
    """Reads SM clocks and throttle reasons through NVML while a region runs (read-only)."""

    def __init__(self, device_index: int):
        self.samples = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._handle = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _run(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(0.001)

    def start(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def summary(self, window):
        """Clocks of the samples taken inside ``window`` (host times) -- and only those."""
        if self._nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"], "samples": 0}
        nv = self._nvml
        inside = [s for s in self.samples if window[0] <= s[0] <= window[1]]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no sample in window"], "samples": 0,
                    "window_ms": (window[1] - window[0]) * 1e3}
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        seen = sorted(name for name, bit in names.items() if any(s[2] & bit for s in inside))
        return {"sm_mhz": int(statistics.median(s[1] for s in inside)), "sm_max_mhz": self.max_mhz,
                "reasons": seen, "samples": len(inside), "window_ms": (window[1] - window[0]) * 1e3}


def make_scan_inputs(rows, T, K, V, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(rows, T, K, device=device, generator=g), dim=-1, eps=1e-6)
    k = torch.nn.functional.normalize(torch.randn(rows, T, K, device=device, generator=g), dim=-1, eps=1e-6)
    v = torch.randn(rows, T, V, device=device, generator=g)
    return k.to(torch.bfloat16), v.to(torch.bfloat16), q.to(torch.bfloat16)


def time_launches(fn, steps, warmup):
    """Mean device time of `steps` calls of fn(i), CUDA events on the current stream."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    events[0].record()
    for i in range(steps):
        fn(warmup + i)
        events[i + 1].record()
    torch.cuda.synchronize()
    return [events[i].elapsed_time(events[i + 1]) for i in range(steps)]


class GraphedStep:
    """`inner` calls of fn(i, stream) captured once as a CUDA graph on a side stream.

    What is measured when the graph is replayed is the GPU executing the launches back to back, not the
    host enqueueing them (a C-ABI call from Python plus its tensor-map lookups costs about as much host
    time as the kernel takes to run)."""

    def __init__(self, fn, inner, eager_warmup=3):
        for i in range(eager_warmup):
            fn(i, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        self.stream = torch.cuda.Stream()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self.stream):
            with torch.cuda.graph(self.graph, stream=self.stream):
                handle = torch.cuda.current_stream().cuda_stream
                for i in range(inner):
                    fn(i, handle)
        torch.cuda.synchronize()

    def time(self, steps, warmup, before_timed=None):
        """Total ms of `steps` replays between one pair of events on the replay stream, after `warmup`
        untimed replays; also the host-time window of the region."""
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                self.graph.replay()
            torch.cuda.synchronize()
            if before_timed is not None:
                before_timed()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record(self.stream)
            for _ in range(steps):
                self.graph.replay()
            e1.record(self.stream)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
        return e0.elapsed_time(e1), (t0, t1)


def time_graph(fn, launches, warmup=3):
    """Mean ms per launch of fn(i, stream): `launches` of them as one graph, replayed once after a warm-up."""
    step = GraphedStep(fn, launches, eager_warmup=warmup)
    total, _ = step.time(1, 1)
    return total / launches


def pinned_input_buffer(nbytes, kind):
    """Page-locked host memory for the input side of the end-to-end leg.  "pinned": torch's pinned allocation.
    "write-combined": cudaHostAlloc with cudaHostAllocWriteCombined -- the CPU writes it once and never reads
    it, the GPUs read it over PCIe without snooping the CPU caches."""
    if kind == "pinned":
        return torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    import ctypes

    from cuda.bindings import runtime as cudart

    err, ptr = cudart.cudaHostAlloc(nbytes, cudart.cudaHostAllocWriteCombined)
    if int(err) != 0:
        raise RuntimeError(f"cudaHostAlloc(write-combined) failed: {err}")
    raw = (ctypes.c_uint8 * nbytes).from_address(int(ptr))
    buffer = torch.frombuffer(raw, dtype=torch.uint8)
    _KEEP_HOST_ALLOCATIONS.append((raw, int(ptr)))               # lives as long as the process
    return buffer


_KEEP_HOST_ALLOCATIONS = []


def max_over_ranks(value, device, world):
    if world <= 1:
        return value
    t = torch.tensor([value], device=device, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def run_engine(args, rank, world, device, numa):
    from rnn_with_grm_b200 import cabi, cuda_ops

    lib = cabi.load()
    if not cuda_ops.load_grm_cuda_extension():
        raise RuntimeError("grm_cuda extension failed to load: " + cuda_ops.get_grm_cuda_runtime_status()["load_error"])
    hbm_peak, tensor_peak, peak_kind = load_peaks()
    rows, T, K, V, decay = CFG2["B"] * CFG2["Hd"], CFG2["T"], CFG2["K"], CFG2["V"], CFG2["decay"]
    tokens_per_batch = CFG2["B"] * T
    inner = args.batches_per_step
    set_bytes = rows * T * (2 * K + 2 * V) * 2
    n_sets = max(2, math.ceil(2.2 * L2_BYTES / set_bytes))
    sets = []
    for s in range(n_sets):
        k, v, q = make_scan_inputs(rows, T, K, V, device, seed=1000 * rank + s)
        sets.append((k, v, q, torch.empty(rows, T, V, device=device, dtype=torch.bfloat16)))
    m_in = torch.zeros(rows, V, K, device=device, dtype=torch.float32)
    m_out = torch.empty_like(m_in)
    # One launch per batch: with 64 rows on 148 SMs the kernel cuts every row along T into two pieces and
    # the second piece derives its start state itself (pre-pass over the first piece's k and v).  The
    # variant with a caller workspace (piece-state kernel + scan, `--with-workspace`) is slower here.
    scratch_bytes = int(lib.grmx_chunk_scan_scratch_bytes(rows, T, K, V, cabi.BF16, cabi.F32))
    scratch = torch.empty(max(scratch_bytes, 16), device=device, dtype=torch.uint8)

    def batch(i, stream):
        k, v, q, o = sets[i % n_sets]
        if args.with_workspace:
            cabi.check(lib.grmx_chunk_scan_fwd_ws(k.data_ptr(), v.data_ptr(), q.data_ptr(), m_in.data_ptr(),
                                                  o.data_ptr(), m_out.data_ptr(), rows, T, K, V, decay, cabi.BF16,
                                                  cabi.F32, cabi.PATH_AUTO, scratch.data_ptr(), scratch_bytes, stream))
        else:
            cabi.check(lib.grmx_chunk_scan_fwd(k.data_ptr(), v.data_ptr(), q.data_ptr(), m_in.data_ptr(),
                                               o.data_ptr(), m_out.data_ptr(), rows, T, K, V, decay, cabi.BF16,
                                               cabi.F32, cabi.PATH_AUTO, stream))

    sampler = ClockSampler(device.index)
    sampler.start()

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # launches are counted where they are enqueued: under capture, once per batch of a step
    before_capture = lib.grmx_launch_count()
    step = GraphedStep(batch, inner, eager_warmup=0)
    launches_per_step = int(lib.grmx_launch_count() - before_capture)
    total_ms, window = step.time(args.steps, args.warmup, barrier)
    barrier()
    total_ms = max_over_ranks(total_ms, device, world)

    # ---- end to end through the public op, host buffers ----
    # Per batch: ONE host->device copy of the packed inputs (k | v | q | start state) from pinned memory,
    # the op, a device-side pack of hidden states and final state, ONE device->host copy into pinned
    # memory.  Batches alternate between two streams with their own buffers, so the copy in of one batch
    # overlaps the copy out of the batch before it (PCIe is full duplex, the GPU has a copy engine per
    # direction); each batch's own chain -- copy in, kernel, copy out -- stays in order on its stream.
    k0, v0, q0, _ = sets[0]
    parts = [k0, v0, q0, m_in]
    part_bytes = [t.numel() * t.element_size() for t in parts]
    in_bytes = sum(part_bytes)
    host_in = pinned_input_buffer(in_bytes, args.host_input)
    at = 0
    for t, n in zip(parts, part_bytes):
        host_in[at:at + n].copy_(t.cpu().contiguous().view(torch.uint8).flatten())
        at += n
    hidden_bytes, state_bytes = rows * T * V * 2, rows * V * K * 4
    out_bytes = hidden_bytes + state_bytes
    lanes = []
    for _ in range(2):
        dev_in = torch.empty(in_bytes, device=device, dtype=torch.uint8)
        views, at = [], 0
        for t, n in zip(parts, part_bytes):
            views.append(dev_in[at:at + n].view(t.dtype).view(t.shape))
            at += n
        lanes.append({"stream": torch.cuda.Stream(device=device), "dev_in": dev_in, "views": views,
                      "dev_out": torch.empty(out_bytes, device=device, dtype=torch.uint8),
                      "host_out": torch.empty(out_bytes, dtype=torch.uint8).pin_memory()})

    def e2e_batch(i):
        lane = lanes[i % 2]
        with torch.cuda.stream(lane["stream"]):
            lane["dev_in"].copy_(host_in, non_blocking=True)
            hidden, state = cuda_ops.cuda_chunk_update(*lane["views"], decay)
            lane["dev_out"][:hidden_bytes].view(torch.bfloat16).view(hidden.shape).copy_(hidden)
            lane["dev_out"][hidden_bytes:].view(torch.float32).view(state.shape).copy_(state)
            lane["host_out"].copy_(lane["dev_out"], non_blocking=True)
            hidden.record_stream(lane["stream"])
            state.record_stream(lane["stream"])

    def time_e2e(batches, warmup):
        for i in range(warmup):
            e2e_batch(i)
        barrier()
        main = torch.cuda.current_stream()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        for lane in lanes:
            lane["stream"].wait_event(e0)
        for i in range(batches):
            e2e_batch(warmup + i)
        for lane in lanes:
            main.wait_stream(lane["stream"])
        e1.record(main)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    e2e_batches = max(8, min(args.steps * 4, 80))
    e2e_ms = time_e2e(e2e_batches, 6)
    barrier()
    e2e_ms = max_over_ranks(e2e_ms, device, world)
    sampler.stop()
    # the packed result of the last batch, checked for sanity: the final state is finite and not zero
    last_state = lanes[(6 + e2e_batches - 1) % 2]["host_out"][hidden_bytes:].view(torch.float32)
    e2e_ok = bool(torch.isfinite(last_state).all() and last_state.abs().max() > 0)

    scale_out = None
    if not args.skip_scale_out:
        scale_out = run_scale_out(args, rank, world, device, hbm_peak)

    if rank != 0:
        return None
    ms_per_step = total_ms / args.steps
    launch_ms = total_ms / (args.steps * max(launches_per_step, 1))
    kernels_per_batch = launches_per_step / inner
    algo_bytes = rows * T * (2 * (2 * K + V) + 2 * V)
    chunk = 64
    algo_flops = rows * T * (2 * chunk * (K + V) + 4 * K * V)
    achieved_gbs = algo_bytes / (launch_ms * kernels_per_batch * 1e-3) / 1e9
    traffic_key = "two_kernel_cut" if kernels_per_batch > 1.5 else "one_launch"
    result = {
        "metric": "memory-path tokens/s",
        "value": world * tokens_per_batch * inner * args.steps / (total_ms * 1e-3),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16 operands, fp32 state and accumulation",
        "data": "synthetic",
        "config": {
            "workload": WORKLOAD,
            "step": f"{inner} consecutive batches per GPU, one scan launch each (one CUDA graph replay)",
            "rows_per_gpu": rows,
            "tokens_per_step_per_gpu": tokens_per_batch * inner,
            "l2": f"inputs rotate over {n_sets} buffer sets ({n_sets * set_bytes / 1e6:.0f} MB > 126 MB L2)",
            "parallelism": f"batch x head rows, one batch stream per GPU on {world} GPU(s), no collective",
            "timing": f"{args.steps} graph replays between one pair of CUDA events on the replay stream, "
                      f"{args.warmup} replays before it untimed",
            "host_numa": numa,
        },
        "timed_region_s": total_ms * 1e-3,
        "row_token_units_per_s": world * rows * T * inner * args.steps / (total_ms * 1e-3),
        "gpu_launches": int(launches_per_step * args.steps),
        "roofline": {
            "bound": "hbm",
            "kernel": "linear-memory scan" + (" (piece-state kernel + scan kernel per batch)" if kernels_per_batch > 1.5
                                              else " (one launch per batch, rows cut along T inside the kernel)"),
            "achieved": achieved_gbs,
            "peak": hbm_peak,
            "unit": "GB/s",
            "frac": achieved_gbs / hbm_peak,
            "peak_source": peak_kind,
            # DRAM bytes of one batch from the ncu capture of this workload (profiles/ncu_figures.json)
            "traffic": profile_figure("scan_kernel_alone_config", traffic_key, "dram_bytes"),
            "traffic_source": "profiles/ncu_figures.json: scan_kernel_alone_config." + traffic_key,
            "algorithmic_bytes_per_launch": algo_bytes,
            "launch_ms": launch_ms * kernels_per_batch,
            "tensor_tflops": algo_flops / (launch_ms * kernels_per_batch * 1e-3) / 1e12,
            "tensor_peak_tflops": tensor_peak,
            "tensor_frac": algo_flops / (launch_ms * kernels_per_batch * 1e-3) / 1e12 / tensor_peak,
        },
        "e2e": {
            "value": world * tokens_per_batch * e2e_batches / (e2e_ms * 1e-3),
            "unit": "tokens/s",
            "h2d_bytes_per_step": int(in_bytes),
            "d2h_bytes_per_step": int(out_bytes),
            "api": "rnn_with_grm_b200.cuda_ops.cuda_chunk_update",
            "step": "one batch: one packed host->device copy, the op, one packed device->host copy",
            "steps": e2e_batches,
            "h2d_gbs_per_gpu": in_bytes * e2e_batches / (e2e_ms * 1e-3) / 1e9,
            "result_read_back_ok": e2e_ok,
        },
        "clocks": sampler.summary(window),
    }
    if scale_out is not None:
        result["scale_out"] = scale_out
    if world == 1 and not args.skip_extras:
        result["cpu_baseline"] = cpu_baseline(budget_s=args.cpu_budget)
        result["other_workloads"] = other_workloads(lib, device, hbm_peak)
    return result


# ---------------------------------------------------------------------------------------------------
# configuration 5: rows sharded over the GPUs, streamed in slabs, sample rows verified over NCCL
# ---------------------------------------------------------------------------------------------------

def run_scale_out(args, rank, world, device, hbm_peak):
    from rnn_with_grm_b200 import scale_out as so
    from rnn_with_grm_b200.sharding import gather_rows, row_range

    shape = so.ScaleOutShape(rows=args.scale_out_rows)
    slab_rows = min(args.slab_rows, max(1, shape.rows // world))
    slabs = so.plan_slabs(shape, rank, world, slab_rows)
    samples = so.sample_rows(shape, rank, world, args.verify_rows)
    host_rows = {row: so.host_row_inputs(shape, row) for row in samples}
    runner = so.SlabRunner(shape, slab_rows, device)
    stream = torch.cuda.current_stream().cuda_stream
    flat = torch.zeros(max(len(samples), 1), so.sample_vector_len(shape), device=device)
    slab_ms, scan_ms, launches = [], [], 0
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    # warm-up on the first slab's data (untimed; sets kernel attributes, fills the tensor-map cache)
    if slabs:
        n = runner.generate(slabs[0][0], slabs[0][1], 0, host_rows)
        runner.segment_means(n)
        for _ in range(2):
            runner.launch(n, stream)
        torch.cuda.synchronize()
    for r0, r1 in slabs:
        n = runner.generate(r0, r1, 0, host_rows)       # input generation: outside the timed region
        runner.segment_means(n)
        torch.cuda.synchronize()
        e0, e1, em = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        launches += runner.launch(n, stream, after_scan=em.record)
        e1.record()
        torch.cuda.synchronize()
        slab_ms.append(e0.elapsed_time(e1))
        scan_ms.append(e0.elapsed_time(em))
        for j, row in enumerate(samples):
            if r0 <= row < r1:
                i = row - r0
                flat[j].copy_(so.pack_sample(runner.hidden[i], runner.m_out[i], runner.fused[i], runner.indices[i]))
    rank_ms = sum(slab_ms)
    total_ms = max_over_ranks(rank_ms, device, world)
    # ---- verification: sample rows of every rank to rank 0 over NCCL, checked against the oracle ----
    n_samples = len(samples)
    counts = torch.tensor([n_samples], device=device)
    if world > 1:
        torch.distributed.all_reduce(counts, op=torch.distributed.ReduceOp.MIN)
    n_each = int(counts.item())                       # the same on every rank (rows divide evenly)
    gathered = flat[:n_each]
    if world > 1 and n_each > 0:
        gathered = gather_rows(flat[:n_each].contiguous(), n_each * world)
    verified = None
    if rank == 0 and n_each > 0:
        all_samples = [row for r in range(world) for row in so.sample_rows(shape, r, world, args.verify_rows)[:n_each]]
        verified = verify_scale_out_rows(shape, all_samples, gathered.cpu())
        verified["gathered_over"] = "nccl all_gather" if world > 1 else "local (one rank)"
    if rank != 0:
        return None
    start, stop = row_range(shape.rows, 0, world)
    scan_bytes = (stop - start) * shape.scan_bytes_per_row()
    return {
        "workload": f"scale-out memory path: {shape.rows} rows (B={shape.rows // shape.heads} x H={shape.heads}) x "
                    f"T={shape.tokens}, d_k=d_v={shape.dim}, segment {shape.segment}, top-k {shape.top_k}, bf16 tokens, "
                    "fp32 state; per slab one scan launch with segment snapshots, routing, fused retrieval",
        "scaling": "strong",
        "n_gpus": world,
        "rows_per_gpu": stop - start,
        "slab_rows": slab_rows,
        "slabs_per_gpu": len(slabs),
        "device_bytes_per_slab": runner.bytes_held(),
        "ms": total_ms,
        "scan_ms_rank0": sum(scan_ms),
        "retrieval_ms_rank0": sum(slab_ms) - sum(scan_ms),
        "tokens_per_s": shape.batch_tokens / (total_ms * 1e-3),
        "row_token_units_per_s": shape.rows * shape.tokens / (total_ms * 1e-3),
        "gpu_launches": launches,
        "per_gpu_scan_gbs": scan_bytes / (total_ms * 1e-3) / 1e9,
        "per_gpu_frac_hbm": scan_bytes / (total_ms * 1e-3) / 1e9 / hbm_peak,
        "per_gpu_path_gbs": so.scale_out_bytes(shape, stop - start) / (total_ms * 1e-3) / 1e9,
        "timing": "CUDA events around each slab's launches on the launching stream, summed per rank, max over ranks; "
                  "inputs are generated on the device between slabs, outside the timed regions",
        "verified": verified,
    }


def verify_scale_out_rows(shape, rows, flat):
    """Sample rows against the oracle: the sequential C scan on the regenerated inputs (hidden states and
    final memory within 2e-2), routing indices bit for bit, fused retrieval within 2e-2."""
    import numpy as np

    import oracle
    from oracle import grm_oracle as go
    from rnn_with_grm_b200 import scale_out as so

    worst = {"hidden": 0.0, "memory": 0.0, "fused": 0.0}
    index_mismatches = 0
    S, L, d = shape.segments, shape.segment, shape.dim
    for j, row in enumerate(rows):
        q, k, v, online = so.host_row_inputs(shape, row)
        hidden, m_out, fused, indices = so.unpack_sample(flat[j], shape)
        qf, kf, vf = (t.float().numpy()[None] for t in (q, k, v))
        memory = np.zeros((1, d, d), dtype=np.float32)
        archive = np.empty((1, S, d, d), dtype=np.float32)
        want_hidden = np.empty((1, shape.tokens, d), dtype=np.float32)
        for s in range(S):
            tok = slice(s * L, (s + 1) * L)
            want_hidden[:, tok], memory = oracle.c_chunk_update(kf[:, tok], vf[:, tok], qf[:, tok], memory, shape.decay)
            archive[:, s] = memory
        seg_q = q.float().view(S, L, d).mean(dim=1).numpy()[None]
        seg_k = k.float().view(S, L, d).mean(dim=1).numpy()[None]
        scores = oracle.c_route_scores(seg_q, seg_k, 1.0)
        want_idx, want_gates = oracle.c_topk_select(scores, shape.top_k, 1.0, np.arange(S, dtype=np.int32))
        want_fused = oracle.c_retrieve_fuse(archive, want_idx, want_gates, seg_q, online.numpy()[None])
        worst["hidden"] = max(worst["hidden"], go.rel_err(hidden.numpy()[None], want_hidden))
        worst["memory"] = max(worst["memory"], go.rel_err(m_out.numpy()[None], memory))
        worst["fused"] = max(worst["fused"], go.rel_err(fused.numpy()[None], want_fused))
        index_mismatches += int((indices.numpy()[None] != want_idx).sum())
    ok = all(v < 2e-2 for v in worst.values()) and index_mismatches == 0
    return {"rows": [int(r) for r in rows], "max_rel_err": worst, "tolerance": 2e-2,
            "routing_index_mismatches": index_mismatches, "ok": bool(ok)}


# ---------------------------------------------------------------------------------------------------
# other workloads (N = 1)
# ---------------------------------------------------------------------------------------------------

def full_occupancy_scan(lib, device, hbm_peak, launches=5):
    """The scan kernel with one batch row per SM and a long sequence: the shape at which the kernel,
    not the number of rows, sets the time.  Timed as one CUDA graph of `launches` launches over
    inputs (0.6 GB) larger than L2."""
    from rnn_with_grm_b200 import cabi

    rows = torch.cuda.get_device_properties(device).multi_processor_count
    T, K, V, decay = 8192, CFG2["K"], CFG2["V"], CFG2["decay"]
    k, v, q = make_scan_inputs(rows, T, K, V, device, seed=7)
    o = torch.empty_like(v)
    m_in = torch.zeros(rows, V, K, device=device)
    m_out = torch.empty_like(m_in)

    def scan(_, stream):
        cabi.check(lib.grmx_chunk_scan_fwd(k.data_ptr(), v.data_ptr(), q.data_ptr(), m_in.data_ptr(), o.data_ptr(),
                                           m_out.data_ptr(), rows, T, K, V, decay, cabi.BF16, cabi.F32,
                                           cabi.PATH_AUTO, stream))

    ms = time_graph(scan, launches)
    nbytes = rows * T * (2 * (2 * K + V) + 2 * V)
    return {"rows": rows, "T": T, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm_peak,
            "bytes": nbytes, "row_tokens_per_s": rows * T / (ms * 1e-3)}


def config2_batches_in_flight(lib, device, hbm_peak, batches=64):
    """The kernel-alone configuration with TWO independent batches in flight: two streams, each replaying its own
    graph of `batches` launches over its own rotating inputs.  The headline times batches one after the other,
    where a launch of 128 CTAs leaves 20 SMs idle and pays its prologue and drain every 24 us; here the second
    stream fills both.  Context for the headline's roofline fraction, not a replacement for it."""
    from rnn_with_grm_b200 import cabi

    rows, T, K, V, decay = CFG2["B"] * CFG2["Hd"], CFG2["T"], CFG2["K"], CFG2["V"], CFG2["decay"]
    set_bytes = rows * T * (2 * K + 2 * V) * 2
    n_sets = max(2, math.ceil(1.2 * L2_BYTES / set_bytes))
    lanes, keep = [], []                                     # the graphs hold raw pointers: the tensors must outlive them
    for lane in range(2):
        sets = []
        for s_ in range(n_sets):
            k, v, q = make_scan_inputs(rows, T, K, V, device, seed=5000 + 100 * lane + s_)
            sets.append((k, v, q, torch.empty(rows, T, V, device=device, dtype=torch.bfloat16)))
        m_in = torch.zeros(rows, V, K, device=device)
        m_out = torch.empty_like(m_in)

        def batch(i, stream, sets=sets, m_in=m_in, m_out=m_out):
            k, v, q, o = sets[i % n_sets]
            cabi.check(lib.grmx_chunk_scan_fwd(k.data_ptr(), v.data_ptr(), q.data_ptr(), m_in.data_ptr(), o.data_ptr(),
                                               m_out.data_ptr(), rows, T, K, V, decay, cabi.BF16, cabi.F32,
                                               cabi.PATH_AUTO, stream))

        keep.append((sets, m_in, m_out))
        lanes.append(GraphedStep(batch, batches, eager_warmup=2))
    replays = 8
    for step in lanes:
        with torch.cuda.stream(step.stream):
            step.graph.replay()
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    ends = [torch.cuda.Event(enable_timing=True) for _ in lanes]
    start.record(torch.cuda.current_stream())
    for step in lanes:
        step.stream.wait_event(start)
    for _ in range(replays):
        for step in lanes:
            with torch.cuda.stream(step.stream):
                step.graph.replay()
    for step, end in zip(lanes, ends):
        end.record(step.stream)
    torch.cuda.synchronize()
    ms = max(start.elapsed_time(end) for end in ends)
    n = 2 * batches * replays
    nbytes = rows * T * (2 * (2 * K + V) + 2 * V)
    del keep
    return {"batches_in_flight": 2, "us_per_batch": ms * 1e3 / n, "tokens_per_s": CFG2["B"] * T * n / (ms * 1e-3),
            "gbs": nbytes * n / ms / 1e6, "frac_hbm": nbytes * n / ms / 1e6 / hbm_peak,
            "timing": "CUDA events on both streams, the later end counts"}


def wide_head_scan(lib, device, hbm_peak, rows=296, T=8192, launches=3):
    """The scan at d_k = d_v = 128 (the head size of the scale-out configuration) alone: `rows` rows of T
    tokens, inputs larger than L2."""
    from rnn_with_grm_b200 import cabi

    d, decay = 128, 0.97
    k, v, q = make_scan_inputs(rows, T, d, d, device, seed=9)
    o = torch.empty_like(v)
    m_in = torch.zeros(rows, d, d, device=device)
    m_out = torch.empty_like(m_in)

    def scan(_, stream):
        cabi.check(lib.grmx_chunk_scan_fwd(k.data_ptr(), v.data_ptr(), q.data_ptr(), m_in.data_ptr(), o.data_ptr(),
                                           m_out.data_ptr(), rows, T, d, d, decay, cabi.BF16, cabi.F32,
                                           cabi.PATH_AUTO, stream))

    for _ in range(30):                                 # ~25 ms of the same work first: clocks settle under the load
        scan(0, torch.cuda.current_stream().cuda_stream)
    ms = time_graph(scan, launches)
    nbytes = rows * T * (2 * (2 * d + d) + 2 * d)
    return {"rows": rows, "T": T, "d": d, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm_peak,
            "bytes": nbytes, "bytes_per_token": 8 * d}


def segment_retrieval(lib, device, hbm_peak, launches=20):
    """The retrieval of ONE config-4 segment with per-token routing: 8 batch rows x 512 tokens choose 4
    of 15 archived segments (512 routing features), then pick, weight, add and normalise the 512-wide
    candidate states (bf16) the dense apply-query has produced.  The two kernels are timed separately,
    each as one CUDA graph of `launches` launches over rotating inputs larger than L2."""
    from rnn_with_grm_b200 import cabi

    B, C, S, D, H, R = CFG4["B"], CFG4["segment"], 15, CFG4["hidden"], CFG4["hidden"], CFG4["top_k"]
    g = torch.Generator(device=device).manual_seed(41)
    keys = torch.randn(B, S, D, device=device, generator=g)
    n_sets = launches
    queries = [torch.randn(B, C, D, device=device, generator=g) for _ in range(n_sets)]           # 8.4 MB each
    states = [torch.randn(B, C, S, H, device=device, generator=g).to(torch.bfloat16) for _ in range(4)]  # 63 MB each
    online = torch.randn(B, C, H, device=device, generator=g).to(torch.bfloat16)
    ln_w, ln_b = torch.ones(H, device=device), torch.zeros(H, device=device)
    idx = torch.empty(B, C, R, device=device, dtype=torch.int64)
    gates = torch.empty(B, C, R, device=device)
    fused = torch.empty(B, C, H, device=device, dtype=torch.bfloat16)

    def route(i, stream):
        cabi.check(lib.grmx_topk_route(queries[i % n_sets].data_ptr(), keys.data_ptr(), None, B, C, S, D, R,
                                       1.0 / math.sqrt(D), 1.0, idx.data_ptr(), gates.data_ptr(), None, stream))

    def select(i, stream):
        cabi.check(lib.grmx_select_fuse(states[i % 4].data_ptr(), idx.data_ptr(), gates.data_ptr(), online.data_ptr(),
                                        ln_w.data_ptr(), ln_b.data_ptr(), 1e-5, fused.data_ptr(), B, C, S, R, H,
                                        cabi.BF16, cabi.FUSE_RESIDUAL_LN, stream))

    route_ms = time_graph(route, launches)
    select_ms = time_graph(select, launches)
    route_bytes = 4 * (B * C * D + B * S * D)
    select_bytes = B * C * (R + 2) * H * 2
    return {"tokens": B * C, "candidates": S, "route_us": route_ms * 1e3, "route_gbs": route_bytes / route_ms / 1e6,
            "select_fuse_us": select_ms * 1e3, "select_fuse_gbs": select_bytes / select_ms / 1e6,
            "select_fuse_frac_hbm": select_bytes / select_ms / 1e6 / hbm_peak}


def layer_retrieval_tc(lib, device, launches=6):
    """The retrieval of one config-4 layer for all tokens at once on the tensor cores: 8 x 8192 tokens, each
    choosing 4 of the slots archived before its segment (16 slots of 512 x 64 bf16), residual + LayerNorm."""
    from rnn_with_grm_b200 import cabi

    B, S, Q, R, H, K = CFG4["B"], 16, CFG4["T"], CFG4["top_k"], CFG4["hidden"], CFG4["K"]
    g = torch.Generator(device=device).manual_seed(43)
    ring = torch.randn(B, S, H, K, device=device, generator=g).to(torch.bfloat16)
    qs = [torch.nn.functional.normalize(torch.randn(B, Q, K, device=device, generator=g), dim=-1).to(torch.bfloat16) for _ in range(3)]
    online = [torch.randn(B, Q, H, device=device, generator=g).to(torch.bfloat16) for _ in range(3)]
    scores = torch.randn(B, Q, S, device=device, generator=g)
    visible = (torch.arange(Q, device=device, dtype=torch.int32) // CFG4["segment"]).to(torch.int32)
    idx = torch.empty(B, Q, R, device=device, dtype=torch.int64)
    gates = torch.empty(B, Q, R, device=device)
    cabi.check(lib.grmx_topk_select(scores.data_ptr(), visible.data_ptr(), B, Q, S, R, 1.0, idx.data_ptr(), gates.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream))
    ln_w, ln_b = torch.ones(H, device=device), torch.zeros(H, device=device)
    out = torch.empty(B, Q, H, device=device, dtype=torch.bfloat16)

    def run(i, stream):
        cabi.check(lib.grmx_retrieve_fuse_tc(ring.data_ptr(), idx.data_ptr(), gates.data_ptr(), qs[i % 3].data_ptr(),
                                             online[i % 3].data_ptr(), ln_w.data_ptr(), ln_b.data_ptr(), 1e-5, out.data_ptr(),
                                             B, S, Q, R, H, K, cabi.FUSE_RESIDUAL_LN, stream))

    ms = time_graph(run, launches)
    live = int((idx >= 0).sum().item())
    flops = 2.0 * live * H * K                       # the products a token needs: R matrices of H x K
    nbytes = B * Q * (K * 2 + 2 * H * 2)             # q in, online in, fused out (the ring stays in L2)
    return {"tokens": B * Q, "slots": S, "us": ms * 1e3, "useful_tflops": flops / (ms * 1e-3) / 1e12,
            "token_gbs": nbytes / ms / 1e6}


def config2_backward(lib, device):
    """Gradients of the config-2 scan (grad_keys, grad_values, grad_queries, grad_memory from grad_hidden
    and grad_memory_out): three scans of the same tensor-core kernel, timed as one CUDA graph."""
    from rnn_with_grm_b200 import cabi

    rows, T, K, V, decay = CFG2["B"] * CFG2["Hd"], CFG2["T"], CFG2["K"], CFG2["V"], CFG2["decay"]
    k, v, q = make_scan_inputs(rows, T, K, V, device, seed=21)
    g = torch.Generator(device=device).manual_seed(22)
    grad_h = torch.randn(rows, T, V, device=device, generator=g).to(torch.bfloat16)
    grad_m = torch.randn(rows, V, K, device=device, generator=g)
    m_in = torch.zeros(rows, V, K, device=device)
    gk, gv, gq, gm = torch.empty_like(k), torch.empty_like(v), torch.empty_like(q), torch.empty_like(m_in)

    def bwd(_, stream):
        cabi.check(lib.grmx_chunk_scan_bwd(grad_h.data_ptr(), grad_m.data_ptr(), k.data_ptr(), v.data_ptr(), q.data_ptr(),
                                           m_in.data_ptr(), gk.data_ptr(), gv.data_ptr(), gq.data_ptr(), gm.data_ptr(),
                                           rows, T, K, V, decay, cabi.BF16, cabi.F32, cabi.PATH_AUTO, stream))

    ms = time_graph(bwd, 5)
    return {"ms": ms, "tokens_per_s": CFG2["B"] * T / (ms * 1e-3)}


def config4_model(device):
    """Config 4 end to end: the four-layer segment-memory language model (hidden 512, d_k 64, segment
    512, top-k 4, vocabulary 32768) over 8 x 8192 token ids, bf16 activations with fp32 state, run by
    the package's own segment loop with random weights under the reference's parameter names, with and
    without the 512 -> 32768 vocabulary projection (which is not part of the memory path)."""
    from rnn_with_grm_b200.segment_memory import GraphedForward, StackedSegmentMemoryRunner, language_model_parameter_shapes

    c4 = CFG4
    g = torch.Generator(device=device).manual_seed(4)
    params = {}
    for name, shape in language_model_parameter_shapes(c4["layers"], c4["hidden"], c4["K"], c4["vocab"], c4["hidden"]).items():
        if name.endswith("layer_norm.weight"):
            t = torch.ones(shape, device=device)
        elif len(shape) == 2 and "embedding" not in name:
            t = (torch.rand(shape, device=device, generator=g) * 2 - 1) * (6.0 / sum(shape)) ** 0.5
        elif "embedding" in name:
            t = torch.randn(shape, device=device, generator=g)
        else:
            t = torch.zeros(shape, device=device)
        params[name] = t.to(torch.bfloat16)
    ids = torch.randint(0, c4["vocab"], (c4["B"], c4["T"]), device=device, generator=g)

    def timed(runner):
        for _ in range(2):
            out, _ = runner.forward(ids, reset_memory=True)
        del out
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0.record()
        for _ in range(reps):
            out, _ = runner.forward(ids, reset_memory=True)
            del out
        e1.record()
        torch.cuda.synchronize()
        eager_ms = e0.elapsed_time(e1) / reps
        # the same forward pass captured as one CUDA graph: on a slow host the eager figure is launch-bound
        graphed = GraphedForward(runner, ids)
        graphed(ids)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            graphed(ids)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps, eager_ms

    kwargs = dict(segment_length=c4["segment"], retrieval_top_k=c4["top_k"], memory_capacity_segments=16,
                  memory_decay=c4["decay"], memory_storage_dtype=torch.float32)
    ms, eager_ms = timed(StackedSegmentMemoryRunner(params, c4["layers"], language_model=True, **kwargs))
    torch.cuda.empty_cache()
    body = StackedSegmentMemoryRunner(params, c4["layers"], language_model=True, **kwargs)
    body.vocabulary_projection = False
    body_ms, _ = timed(body)
    torch.cuda.empty_cache()
    return {"ms": ms, "tokens_per_s": c4["B"] * c4["T"] / (ms * 1e-3), "eager_ms": eager_ms,
            "ms_without_vocabulary_projection": body_ms,
            "tokens_per_s_without_vocabulary_projection": c4["B"] * c4["T"] / (body_ms * 1e-3),
            "layers": c4["layers"], "hidden": c4["hidden"], "segments": c4["T"] // c4["segment"],
            "dtype": "bf16 activations, fp32 state", "timing": "forward pass captured as one CUDA graph"}


def config3_retrieval(lib, device, hbm_peak):
    """Config 3: one query per segment, causal top-4 over 32 archived 64 x 64 fp32 matrices per row, 128
    rows.  Every launch reads another archive of a rotation larger than L2, so the matrices come from HBM."""
    from rnn_with_grm_b200 import cabi

    out = {}
    stream = torch.cuda.current_stream().cuda_stream
    rows, S, K, V, top_k = CFG3["B"] * CFG3["Hd"], CFG3["T"] // CFG3["segment"], CFG3["K"], CFG3["V"], CFG3["top_k"]
    g = torch.Generator(device=device).manual_seed(3)
    qn = torch.nn.functional.normalize(torch.randn(rows, CFG3["T"], K, device=device, generator=g), dim=-1)
    kn = torch.nn.functional.normalize(torch.randn(rows, CFG3["T"], K, device=device, generator=g), dim=-1)
    seg_q = qn.view(rows, S, CFG3["segment"], K).mean(dim=2).contiguous()
    seg_k = kn.view(rows, S, CFG3["segment"], K).mean(dim=2).contiguous()
    del qn, kn
    n_arch = 6                                                         # 6 x 67 MB = 403 MB > 3 x L2
    archives = [torch.randn(rows, S, V, K, device=device, generator=g) for _ in range(n_arch)]
    online = torch.randn(rows, S, V, device=device, generator=g)
    visible = torch.arange(S, device=device, dtype=torch.int32)
    idx = torch.empty(rows, S, top_k, device=device, dtype=torch.int64)
    gates = torch.empty(rows, S, top_k, device=device, dtype=torch.float32)
    fused = torch.empty(rows, S, V, device=device, dtype=torch.float32)
    gathered = torch.empty(rows, S, top_k, V, K, device=device, dtype=torch.float32)

    def route(_):
        cabi.check(lib.grmx_topk_route(seg_q.data_ptr(), seg_k.data_ptr(), visible.data_ptr(), rows, S, S, K, top_k,
                                       1.0, 1.0, idx.data_ptr(), gates.data_ptr(), None, stream))

    def fuse(i):
        cabi.check(lib.grmx_retrieve_fuse(archives[i % n_arch].data_ptr(), idx.data_ptr(), gates.data_ptr(),
                                          seg_q.data_ptr(), online.data_ptr(), None, None, 1e-5, fused.data_ptr(),
                                          rows, S, S, top_k, V, K, cabi.FUSE_RESIDUAL_LN, stream))

    def gather(i):
        cabi.check(lib.grmx_batched_gather(archives[i % n_arch].data_ptr(), idx.data_ptr(), gathered.data_ptr(), rows, S,
                                           S * top_k, V * K, 4, stream))

    route(0)
    torch.cuda.synchronize()
    live = int((idx >= 0).sum().item())
    distinct = int(torch.zeros(rows, S, device=device).scatter_(1, idx.clamp_min(0).view(rows, -1),
                                                                (idx >= 0).float().view(rows, -1)).sum().item())
    mat_bytes = V * K * 4
    # Routing reads 2 MB per launch and runs for a few microseconds, less than the host needs to enqueue a launch
    # from Python: it is timed as one graph of launches, each on another copy of its inputs (160 MB in turn, more
    # than L2 holds).
    n_rot = 80
    rot_q = [seg_q.clone() for _ in range(n_rot)]
    rot_k = [seg_k.clone() for _ in range(n_rot)]

    def route_graphed(i, handle):
        cabi.check(lib.grmx_topk_route(rot_q[i % n_rot].data_ptr(), rot_k[i % n_rot].data_ptr(), visible.data_ptr(), rows,
                                       S, S, K, top_k, 1.0, 1.0, idx.data_ptr(), gates.data_ptr(), None, handle))

    out["cfg3_topk_route_ms"] = time_graph(route_graphed, 2 * n_rot)
    out["cfg3_topk_route_timing"] = f"one CUDA graph of {2 * n_rot} launches over {n_rot} copies of the inputs"
    del rot_q, rot_k
    fuse_ms = statistics.mean(time_launches(fuse, 24, 6))
    fuse_bytes = live * mat_bytes + rows * S * V * 8
    fuse_dram = distinct * mat_bytes + rows * S * V * 8               # a matrix selected by several queries is read from HBM once
    out["cfg3_retrieve_fuse"] = {
        "ms": fuse_ms, "bytes": fuse_bytes, "algorithmic_gbs": fuse_bytes / fuse_ms / 1e6,
        "frac_hbm_algorithmic": fuse_bytes / fuse_ms / 1e6 / hbm_peak,
        "distinct_bytes": fuse_dram, "distinct_gbs": fuse_dram / fuse_ms / 1e6,
        "frac_hbm_distinct": fuse_dram / fuse_ms / 1e6 / hbm_peak,
        "dram_bytes_ncu": profile_figure("retrieve_fuse_config3", "dram_bytes"),
        "note": "the slot-major kernel reads every chosen matrix once per batch row (the distinct bytes); the "
                "algorithmic figure counts a matrix once per query that selects it, as the reference's gather does, and "
                "is a figure of merit here, not a bandwidth",
    }
    gather_ms = statistics.mean(time_launches(gather, 24, 6))
    gather_bytes = live * mat_bytes + rows * S * top_k * mat_bytes    # reads of live slots + writes of every slot
    gather_dram = distinct * mat_bytes + rows * S * top_k * mat_bytes
    out["cfg3_gather"] = {
        "ms": gather_ms, "bytes": gather_bytes, "algorithmic_gbs": gather_bytes / gather_ms / 1e6,
        "frac_hbm_algorithmic": gather_bytes / gather_ms / 1e6 / hbm_peak,
        "distinct_bytes": gather_dram, "distinct_gbs": gather_dram / gather_ms / 1e6,
        "frac_hbm_distinct": gather_dram / gather_ms / 1e6 / hbm_peak,
        "dram_bytes_ncu": profile_figure("batched_gather_config3", "dram_bytes"),
        "note": "algorithmic bytes count a matrix once per query that selects it; re-selected matrices of a row hit "
                "L2, so the distinct figure is the one to hold against the HBM roofline",
    }
    for key in ("cfg3_retrieve_fuse", "cfg3_gather"):
        ncu = out[key]["dram_bytes_ncu"]
        out[key]["dram_gbs_ncu"] = None if ncu is None else ncu / out[key]["ms"] / 1e6
    out["cfg3_tokens_per_s_route_plus_fuse"] = CFG3["B"] * CFG3["T"] / ((out["cfg3_topk_route_ms"] + fuse_ms) * 1e-3)
    out["cfg3_archive_rotation"] = f"{n_arch} archives of {rows * S * mat_bytes / 1e6:.0f} MB, one per launch in turn"
    return out


def other_workloads(lib, device, hbm_peak):
    """Kernel-timed figures for the other configurations."""
    out = {}
    out["full_occupancy_scan"] = full_occupancy_scan(lib, device, hbm_peak)
    out["wide_head_scan"] = wide_head_scan(lib, device, hbm_peak)
    out["cfg2_backward"] = config2_backward(lib, device)
    out["cfg2_two_batches_in_flight"] = config2_batches_in_flight(lib, device, hbm_peak)
    torch.cuda.empty_cache()
    torch.cuda.empty_cache()
    out["cfg4_model"] = config4_model(device)
    out["cfg4_segment_retrieval"] = segment_retrieval(lib, device, hbm_peak)
    out["cfg4_layer_retrieval_tc"] = layer_retrieval_tc(lib, device)
    torch.cuda.empty_cache()
    out.update(config3_retrieval(lib, device, hbm_peak))
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------------
# the reference's CPU implementation (cpu_baseline, --impl reference)
# ---------------------------------------------------------------------------------------------------

def config2_host_inputs(seed=0):
    rows, T, K, V = CFG2["B"] * CFG2["Hd"], CFG2["T"], CFG2["K"], CFG2["V"]
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(rows, T, K, generator=g), dim=-1, eps=1e-6)
    k = torch.nn.functional.normalize(torch.randn(rows, T, K, generator=g), dim=-1, eps=1e-6)
    v = torch.randn(rows, T, V, generator=g)
    return k, v, q, torch.zeros(rows, V, K)


class ReferenceCpuPath:
    """The reference's chunk update on CPU tensors, one config-2 batch per call.

    ``kind == "reference"``: ``grm.core.cuda_ops.cuda_chunk_update`` imported from the staged reference
    package; with CPU tensors its dispatch takes the vectorised PyTorch math (grm/core/cuda_ops.py:117-135,
    218-254, 367), driven per call of ``tokens_per_call`` tokens with the state carried, as the reference's
    segment loop drives it.  Without the staged package: the reference's compiled sequential C++ op
    (grm/csrc/grm_cuda.cpp:46-90) when it was built, else the C restatement (``kind == "port"``).
    """

    def __init__(self):
        import oracle

        self.cores = os.cpu_count() or 1
        try:
            self.cores = len(os.sched_getaffinity(0))
        except AttributeError:
            pass
        torch.set_num_threads(self.cores)
        self.k, self.v, self.q, self.m = config2_host_inputs()
        self.decay = CFG2["decay"]
        self.fn = None
        self.tokens_per_call = None
        staged = oracle.reference_python()
        self.cpp = oracle.reference_ops()
        if staged is not None:
            sys.dont_write_bytecode = True
            if str(staged) not in sys.path:
                sys.path.insert(0, str(staged))
            from grm.core.cuda_ops import cuda_chunk_update
            self.fn = cuda_chunk_update
            self.kind = "reference"
            self.what = "grm.core.cuda_ops.cuda_chunk_update on CPU tensors (the reference's default CPU path: vectorised PyTorch math)"
        elif self.cpp is not None:
            self.kind = "reference"
            self.what = "grm::chunk_update_forward, the reference's compiled sequential CPU op (grm/csrc/grm_cuda.cpp:46-90)"
        else:
            self.kind = "port"
            self.what = "C restatement of the sequential scan (oracle/grm_oracle.c)"

    def one_batch(self, tokens_per_call=None):
        """Seconds for all 64 rows x 2048 tokens."""
        import numpy as np

        import oracle

        t0 = time.perf_counter()
        if self.fn is not None:
            memory = self.m
            with torch.no_grad():
                for s0 in range(0, CFG2["T"], tokens_per_call):
                    s1 = s0 + tokens_per_call
                    _, memory = self.fn(self.k[:, s0:s1], self.v[:, s0:s1], self.q[:, s0:s1], memory, self.decay)
        elif self.cpp is not None:
            self.cpp.chunk_update_forward(self.k, self.v, self.q, self.m, self.decay)
        else:
            oracle.c_chunk_update(*(np.ascontiguousarray(t.numpy()) for t in (self.k, self.v, self.q, self.m)), self.decay)
        return time.perf_counter() - t0

    def pick_call_size(self):
        if self.fn is None:
            return None
        best = None
        for size in (64, 128):
            self.one_batch(size)
            dt = min(self.one_batch(size) for _ in range(2))
            if best is None or dt < best[1]:
                best = (size, dt)
        self.tokens_per_call = best[0]
        return best[0]

    def cpp_op_seconds(self):
        if self.cpp is None:
            return None
        t0 = time.perf_counter()
        self.cpp.chunk_update_forward(self.k, self.v, self.q, self.m, self.decay)
        return time.perf_counter() - t0


def cpu_baseline(budget_s):
    ref = ReferenceCpuPath()
    size = ref.pick_call_size()
    ref.one_batch(size)
    times, spent = [], 0.0
    while spent < budget_s and len(times) < 400:
        dt = ref.one_batch(size)
        times.append(dt)
        spent += dt
    dt = statistics.median(times)
    tokens = CFG2["B"] * CFG2["T"]
    out = {"value": tokens / dt, "unit": "tokens/s", "cores": ref.cores, "kind": ref.kind,
           "sample": f"all 64 (b,h) rows x T=2048 per pass, fp32, median of {len(times)} passes ({spent:.1f} s); {ref.what}"
                     + (f", {size} tokens per call" if size else ""),
           "seconds": dt}
    cpp = ref.cpp_op_seconds()
    if cpp is not None and ref.fn is not None:
        out["compiled_cpp_op"] = {"value": tokens / cpp, "unit": "tokens/s", "seconds": cpp,
                                  "what": "grm::chunk_update_forward (grm/csrc/grm_cuda.cpp:46-90), one call over T=2048"}
    return out


def run_reference(args, rank, world):
    if rank != 0:
        return None
    ref = ReferenceCpuPath()
    size = ref.pick_call_size()
    for _ in range(max(1, min(args.warmup, 3))):
        ref.one_batch(size)
    times = [ref.one_batch(size) for _ in range(args.steps)]
    total = sum(times)
    tokens = CFG2["B"] * CFG2["T"]
    value = tokens * args.steps / total
    cpu = {"value": value, "unit": "tokens/s", "cores": ref.cores, "kind": ref.kind,
           "sample": f"one batch (64 (b,h) rows x T=2048) per step, fp32, {args.steps} steps; {ref.what}"
                     + (f", {size} tokens per call" if size else "")}
    cpp = ref.cpp_op_seconds()
    if cpp is not None and ref.fn is not None:
        cpu["compiled_cpp_op"] = {"value": tokens / cpp, "unit": "tokens/s", "seconds": cpp,
                                  "what": "grm::chunk_update_forward (grm/csrc/grm_cuda.cpp:46-90), one call over T=2048"}
    return {
        "impl": "reference",
        "metric": "memory-path tokens/s",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "step": "one batch on the host cores (a bounded sample of the engine arm's step)"},
        "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=["engine", "reference"], default="engine")
    parser.add_argument("--batches-per-step", type=int, default=128,
                        help="batches (scan launches) per step; the batches of a step are one CUDA graph")
    parser.add_argument("--skip-extras", action="store_true",
                        help="no CPU baseline and no other workloads (small footprint for profiling)")
    parser.add_argument("--skip-scale-out", action="store_true", help="do not run the sharded configuration 5")
    parser.add_argument("--scale-out-rows", type=int, default=4096, help="rows of configuration 5 (all GPUs together)")
    parser.add_argument("--slab-rows", type=int, default=296,
                        help="rows a GPU holds at a time in configuration 5 (296 rows x 2 value blocks = 4 CTAs per SM of a B200)")
    parser.add_argument("--verify-rows", type=int, default=2, help="rows per rank checked against the oracle")
    parser.add_argument("--cpu-budget", type=float, default=10.0, help="seconds of CPU work for cpu_baseline")
    parser.add_argument("--host-input", choices=["pinned", "write-combined"], default="pinned",
                        help="how the host buffer of the end-to-end leg's inputs is allocated")
    parser.add_argument("--with-workspace", action="store_true",
                        help="time the two-kernel variant of the cut (piece-state kernel + scan over a caller workspace)")
    parser.add_argument("--only", choices=["full-occupancy", "wide-head", "config4", "segment-retrieval", "layer-retrieval",
                                           "config3", "scale-out"],
                        help="run one of the other workloads alone and print its figures (for profiling)")
    # earlier spellings of --only, kept so that the commands recorded under profiles/ still run as written
    for old, new in (("--full-occupancy-only", "full-occupancy"), ("--config4-only", "config4"),
                     ("--segment-retrieval-only", "segment-retrieval")):
        parser.add_argument(old, dest="only", action="store_const", const=new, help=argparse.SUPPRESS)
    args = parser.parse_args(argv)
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 1)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")

    if args.impl == "reference":
        result = run_reference(args, rank, world)
        if result is not None:
            print(json.dumps(result), flush=True)
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    numa = bind_to_gpu_numa_node(local_rank)          # before the first pinned allocation
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    try:
        if args.only is not None:
            from rnn_with_grm_b200 import cabi, cuda_ops

            if not cuda_ops.load_grm_cuda_extension():
                raise RuntimeError("grm_cuda extension failed to load: " + cuda_ops.get_grm_cuda_runtime_status()["load_error"])
            lib, peak = cabi.load(), load_peaks()[0]
            if args.only == "full-occupancy":
                out = {"full_occupancy_scan": full_occupancy_scan(lib, device, peak)}
            elif args.only == "wide-head":
                out = {"wide_head_scan": wide_head_scan(lib, device, peak)}
            elif args.only == "config4":
                out = {"cfg4_model": config4_model(device)}
            elif args.only == "segment-retrieval":
                out = {"cfg4_segment_retrieval": segment_retrieval(lib, device, peak, launches=4)}
            elif args.only == "layer-retrieval":
                out = {"cfg4_layer_retrieval_tc": layer_retrieval_tc(lib, device)}
            elif args.only == "config3":
                out = config3_retrieval(lib, device, peak)
            else:
                out = {"scale_out": run_scale_out(args, rank, world, device, peak)}
            if rank == 0:
                print(json.dumps(out), flush=True)
            return 0
        result = run_engine(args, rank, world, device, numa)
        if result is not None:
            print(json.dumps(result), flush=True)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
