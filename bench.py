#!/usr/bin/env python
"""Benchmark of the segment-memory hot path: tokens/s of the chunked linear-memory
update + query on the kernel-alone configuration (B=8, H=8, T=2048, d_k=d_v=64, bf16
inputs, fp32 carried state), one such batch per GPU (weak scaling, no collective on the
data path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl engine|reference]

N > 1 is launched by ``python -m torch.distributed.run --nproc-per-node N ... bench.py
--gpus N``; rank 0 prints ONE JSON line.  Keys beyond the base contract:

* ``roofline``      -- the scan kernel against the HBM roofline (algorithmic bytes per launch
                       / mean launch time from CUDA events on the launching stream), with the
                       tensor-pipe figures beside it;
* ``cpu_baseline``  -- the reference's own CPU implementation timed on this host's cores;
* ``e2e``           -- the same metric through ``cuda_ops.cuda_chunk_update`` with pinned host
                       buffers, host<->device copies inside the timed region;
* ``other_workloads`` -- top-k retrieval + fusion (config 3) and a slab of the scale-out
                       config 5, kernel-timed, N=1 only.

``--impl reference`` times the reference's CPU code (``oracle/_ref`` when it was built, else
the C restatement) on the same workload; it is the only arm that executes ``oracle/``.
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
CFG5_SLAB = dict(rows=256, T=32768, K=128, V=128, decay=0.97)   # 256 of the 4096 (b,h) rows of config 5
L2_BYTES = 126 * 1024 * 1024


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), float(data["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


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
            time.sleep(0.002)

    def start(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def summary(self, windows):
        if self._nvml is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        nv = self._nvml
        inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in windows)] or self.samples
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        seen = sorted(name for name, bit in names.items() if any(s[2] & bit for s in inside))
        return {"sm_mhz": int(statistics.median(s[1] for s in inside)), "sm_max_mhz": self.max_mhz,
                "reasons": seen, "samples": len(inside)}


def make_scan_inputs(rows, T, K, V, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(rows, T, K, device=device, generator=g), dim=-1, eps=1e-6)
    k = torch.nn.functional.normalize(torch.randn(rows, T, K, device=device, generator=g), dim=-1, eps=1e-6)
    v = torch.randn(rows, T, V, device=device, generator=g)
    return k.to(torch.bfloat16), v.to(torch.bfloat16), q.to(torch.bfloat16)


def time_launches(fn, steps, warmup, before_timed=None):
    """Mean and total device time of `steps` calls of fn(i), CUDA events on the current stream."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if before_timed is not None:
        before_timed()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    t0 = time.perf_counter()
    events[0].record()
    for i in range(steps):
        fn(warmup + i)
        events[i + 1].record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    per = [events[i].elapsed_time(events[i + 1]) for i in range(steps)]
    return events[0].elapsed_time(events[steps]), per, (t0, t1)


def time_graph(fn, steps, warmup, before_timed=None):
    """Device time of `steps` calls of fn(i, stream) replayed as ONE CUDA graph.

    The calls are enqueued once, under stream capture, and the timed region is a single graph
    launch bracketed by CUDA events on the launching stream: what is measured is the GPU
    executing the steps back to back, not the host enqueueing them (on a slow host core a C-ABI
    call plus its tensor-map encodes costs about as much as the kernels take to run).
    Warm-up: `warmup` eager calls, then one untimed replay of the whole graph.
    """
    for i in range(warmup):
        fn(i, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            handle = torch.cuda.current_stream().cuda_stream
            for i in range(steps):
                fn(warmup + i, handle)
        graph.replay()
        torch.cuda.synchronize()
        if before_timed is not None:
            before_timed()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(side)
        graph.replay()
        e1.record(side)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
    total = e0.elapsed_time(e1)
    return total, [total / steps] * steps, (t0, t1)


def run_engine(args, rank, world, device):
    from rnn_with_grm_b200 import cabi, cuda_ops

    lib = cabi.load()
    if not cuda_ops.load_grm_cuda_extension():
        raise RuntimeError("grm_cuda extension failed to load: " + cuda_ops.get_grm_cuda_runtime_status()["load_error"])
    hbm_peak, tensor_peak, peak_kind = load_peaks()
    rows, T, K, V, decay = CFG2["B"] * CFG2["Hd"], CFG2["T"], CFG2["K"], CFG2["V"], CFG2["decay"]
    tokens_per_step = CFG2["B"] * T
    set_bytes = rows * T * (2 * K + 2 * V) * 2
    n_sets = max(2, math.ceil(2.2 * L2_BYTES / set_bytes))
    sets = []
    for s in range(n_sets):
        k, v, q = make_scan_inputs(rows, T, K, V, device, seed=1000 * rank + s)
        sets.append((k, v, q, torch.empty(rows, T, V, device=device, dtype=torch.bfloat16)))
    m_in = torch.zeros(rows, V, K, device=device, dtype=torch.float32)
    m_out = torch.empty_like(m_in)
    # One launch per step: with 64 rows on 148 SMs the kernel cuts every row along T into two pieces
    # and the second piece derives its start state itself (pre-pass over the first piece's k and v).
    # The variant with a caller workspace (piece-state kernel + scan, `--with-workspace`) is slower
    # at this shape: two launches' worth of fixed cost.
    scratch_bytes = int(lib.grmx_chunk_scan_scratch_bytes(rows, T, K, V, cabi.BF16, cabi.F32))
    scratch = torch.empty(max(scratch_bytes, 16), device=device, dtype=torch.uint8)

    def step(i, stream):
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

    # launches are counted where they are enqueued: the warm-up calls, then the captured steps
    before_capture = lib.grmx_launch_count()
    total_ms, per_ms, window = time_graph(step, args.steps, args.warmup, barrier)
    launches = lib.grmx_launch_count() - before_capture
    launches = launches * args.steps // (args.steps + args.warmup)       # the captured steps' share
    barrier()
    if world > 1:
        t = torch.tensor([total_ms], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        total_ms = float(t.item())

    # ---- end to end through the public op, host buffers ----
    # Every step copies its inputs from pinned host memory, runs the op and copies hidden states and
    # final state back.  Steps alternate between two streams with their own device buffers, so the
    # input copy of one step overlaps the output copy of the step before it (PCIe is full duplex and
    # the GPU has separate copy engines for the two directions); each step's own chain -- copy in,
    # kernel, copy out -- stays in order on its stream.
    k0, v0, q0, _ = sets[0]
    host_in = [t.cpu().pin_memory() for t in (k0, v0, q0)] + [m_in.cpu().pin_memory()]
    lanes = []
    for _ in range(2):
        lanes.append({"stream": torch.cuda.Stream(device=device),
                      "dev_in": [torch.empty_like(t, device=device) for t in host_in],
                      "host_hidden": torch.empty(rows, T, V, dtype=torch.bfloat16).pin_memory(),
                      "host_state": torch.empty(rows, V, K, dtype=torch.float32).pin_memory()})
    host_hidden, host_state = lanes[0]["host_hidden"], lanes[0]["host_state"]

    def e2e_step(i):
        lane = lanes[i % 2]
        with torch.cuda.stream(lane["stream"]):
            for d, h in zip(lane["dev_in"], host_in):
                d.copy_(h, non_blocking=True)
            hidden, state = cuda_ops.cuda_chunk_update(*lane["dev_in"], decay)
            lane["host_hidden"].copy_(hidden, non_blocking=True)
            lane["host_state"].copy_(state, non_blocking=True)
            hidden.record_stream(lane["stream"])
            state.record_stream(lane["stream"])

    def time_e2e(steps, warmup):
        for i in range(warmup):
            e2e_step(i)
        barrier()
        main = torch.cuda.current_stream()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(main)
        for lane in lanes:
            lane["stream"].wait_event(e0)
        for i in range(steps):
            e2e_step(warmup + i)
        for lane in lanes:
            main.wait_stream(lane["stream"])
        e1.record(main)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        return e0.elapsed_time(e1), (t0, t1)

    e2e_steps = max(4, min(args.steps, 20))
    e2e_ms, e2e_window = time_e2e(e2e_steps, max(4, min(args.warmup, 6)))
    barrier()
    if world > 1:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_ms = float(t.item())
    sampler.stop()

    if rank != 0:
        return None
    ms_per_step = total_ms / args.steps
    launch_ms = statistics.mean(per_ms)
    kernels_per_step = launches / max(args.steps, 1)
    algo_bytes = rows * T * (2 * (2 * K + V) + 2 * V)
    chunk = 64
    algo_flops = rows * T * (2 * chunk * (K + V) + 4 * K * V)
    achieved_gbs = algo_bytes / (launch_ms * 1e-3) / 1e9
    result = {
        "metric": "memory-path tokens/s",
        "value": world * tokens_per_step * args.steps / (total_ms * 1e-3),
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
            "workload": "chunked linear-memory update + query kernel alone: B=8 H=8 T=2048 d_k=64 d_v=64, "
                        "decay 0.97, zero start state, one batch per GPU",
            "rows_per_gpu": rows,
            "tokens_per_step_per_gpu": tokens_per_step,
            "l2": f"inputs rotate over {n_sets} buffer sets ({n_sets * set_bytes / 1e6:.0f} MB > 126 MB L2)",
            "parallelism": f"batch x head rows sharded over {world} GPU(s), no collective",
            "timing": "the timed steps are captured once into a CUDA graph; the timed region is one replay",
        },
        "row_token_units_per_s": world * rows * T * args.steps / (total_ms * 1e-3),
        "gpu_launches": int(launches),
        "roofline": {
            "bound": "hbm",
            "kernel": "linear-memory scan" + (" (piece-state kernel + scan kernel per step)" if kernels_per_step > 1.5
                                              else " (one launch per step, rows cut along T inside the kernel)"),
            "achieved": achieved_gbs,
            "peak": hbm_peak,
            "unit": "GB/s",
            "frac": achieved_gbs / hbm_peak,
            "peak_source": peak_kind,
            # DRAM bytes of one step from the ncu captures of this workload (profiles/).  One launch:
            # 51.5 MB read + 1.9 MB written (the output is still in L2 when the kernel ends).  Two-kernel
            # cut: scan 53.6 MB read + 2.4 MB written, piece-state kernel 16.8 MB read.
            "traffic": 72783616 if kernels_per_step > 1.5 else 53354240,
            "algorithmic_bytes_per_launch": algo_bytes,
            "launch_ms": launch_ms,
            "tensor_tflops": algo_flops / (launch_ms * 1e-3) / 1e12,
            "tensor_peak_tflops": tensor_peak,
            "tensor_frac": algo_flops / (launch_ms * 1e-3) / 1e12 / tensor_peak,
        },
        "e2e": {
            "value": world * tokens_per_step * e2e_steps / (e2e_ms * 1e-3),
            "unit": "tokens/s",
            "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in host_in)),
            "d2h_bytes_per_step": int(host_hidden.numel() * 2 + host_state.numel() * 4),
            "api": "rnn_with_grm_b200.cuda_ops.cuda_chunk_update",
            "steps": e2e_steps,
        },
        "clocks": sampler.summary([window, e2e_window]),
    }
    if world == 1 and not args.skip_extras:
        result["cpu_baseline"] = cpu_baseline(sample_rows=rows, reps=3)
        result["other_workloads"] = other_workloads(lib, device, hbm_peak)
    return result


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

    total_ms, _, _ = time_graph(scan, launches, 3)
    ms = total_ms / launches
    nbytes = rows * T * (2 * (2 * K + V) + 2 * V)
    return {"rows": rows, "T": T, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm_peak,
            "bytes": nbytes, "row_tokens_per_s": rows * T / (ms * 1e-3)}


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

    route_ms = time_graph(route, launches, 3)[0] / launches
    select_ms = time_graph(select, launches, 3)[0] / launches
    route_bytes = 4 * (B * C * D + B * S * D)
    select_bytes = B * C * (R + 2) * H * 2
    return {"tokens": B * C, "candidates": S, "route_us": route_ms * 1e3, "route_gbs": route_bytes / route_ms / 1e6,
            "select_fuse_us": select_ms * 1e3, "select_fuse_gbs": select_bytes / select_ms / 1e6,
            "select_fuse_frac_hbm": select_bytes / select_ms / 1e6 / hbm_peak}


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

    launches = 5
    total_ms, _, _ = time_graph(bwd, launches, 3)
    ms = total_ms / launches
    return {"ms": ms, "tokens_per_s": CFG2["B"] * T / (ms * 1e-3)}


def config4_model(device):
    """Config 4 end to end: the four-layer segment-memory language model (hidden 512, d_k 64, segment
    512, top-k 4, vocabulary 32768) over 8 x 8192 token ids, bf16 activations with fp32 state, run by
    the package's own segment loop with random weights under the reference's parameter names.  The
    figure includes the projections (cuBLAS) and the 512 -> 32768 output layer."""
    from rnn_with_grm_b200.segment_memory import StackedSegmentMemoryRunner, language_model_parameter_shapes

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
    runner = StackedSegmentMemoryRunner(params, c4["layers"], language_model=True, segment_length=c4["segment"],
                                        retrieval_top_k=c4["top_k"], memory_capacity_segments=16, memory_decay=c4["decay"])
    ids = torch.randint(0, c4["vocab"], (c4["B"], c4["T"]), device=device, generator=g)
    for _ in range(2):
        logits, _ = runner.forward(ids, reset_memory=True)
    del logits
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    e0.record()
    for _ in range(reps):
        logits, _ = runner.forward(ids, reset_memory=True)
        del logits
    e1.record()
    torch.cuda.synchronize()
    eager_ms = e0.elapsed_time(e1) / reps
    # the same forward pass captured as one CUDA graph: on a slow host the eager figure is launch-bound
    from rnn_with_grm_b200.segment_memory import GraphedForward
    graphed = GraphedForward(runner, ids)
    graphed(ids)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        graphed(ids)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    return {"ms": ms, "tokens_per_s": c4["B"] * c4["T"] / (ms * 1e-3), "eager_ms": eager_ms, "layers": c4["layers"],
            "hidden": c4["hidden"], "segments": c4["T"] // c4["segment"], "dtype": "bf16 activations, fp32 state",
            "timing": "forward pass captured as one CUDA graph"}


def other_workloads(lib, device, hbm_peak):
    """Kernel-timed figures for the retrieval path (config 3) and a config-5 slab."""
    from rnn_with_grm_b200 import cabi

    out = {}
    out["full_occupancy_scan"] = full_occupancy_scan(lib, device, hbm_peak)
    out["cfg2_backward"] = config2_backward(lib, device)
    out["cfg4_model"] = config4_model(device)
    out["cfg4_segment_retrieval"] = segment_retrieval(lib, device, hbm_peak)
    torch.cuda.empty_cache()
    stream = torch.cuda.current_stream().cuda_stream
    # ---- config 3: one query per segment, causal top-4 over 32 archived 64x64 fp32 matrices ----
    rows, S, K, V, top_k = CFG3["B"] * CFG3["Hd"], CFG3["T"] // CFG3["segment"], CFG3["K"], CFG3["V"], CFG3["top_k"]
    g = torch.Generator(device=device).manual_seed(3)
    qn = torch.nn.functional.normalize(torch.randn(rows, CFG3["T"], K, device=device, generator=g), dim=-1)
    kn = torch.nn.functional.normalize(torch.randn(rows, CFG3["T"], K, device=device, generator=g), dim=-1)
    seg_q = qn.view(rows, S, CFG3["segment"], K).mean(dim=2).contiguous()
    seg_k = kn.view(rows, S, CFG3["segment"], K).mean(dim=2).contiguous()
    del qn, kn
    archives = [torch.randn(rows, S, V, K, device=device, generator=g) for _ in range(3)]   # 3 x 67 MB
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
        cabi.check(lib.grmx_retrieve_fuse(archives[i % 3].data_ptr(), idx.data_ptr(), gates.data_ptr(),
                                          seg_q.data_ptr(), online.data_ptr(), None, None, 1e-5, fused.data_ptr(),
                                          rows, S, S, top_k, V, K, cabi.FUSE_RESIDUAL_LN, stream))

    def gather(i):
        cabi.check(lib.grmx_batched_gather(archives[i % 3].data_ptr(), idx.data_ptr(), gathered.data_ptr(), rows, S,
                                           S * top_k, V * K, 4, stream))

    route(0)
    torch.cuda.synchronize()
    live = int((idx >= 0).sum().item())
    mat_bytes = V * K * 4
    _, per, _ = time_launches(route, 20, 3)
    out["cfg3_topk_route_ms"] = statistics.mean(per)
    _, per, _ = time_launches(fuse, 20, 3)
    fuse_ms = statistics.mean(per)
    fuse_bytes = live * mat_bytes + rows * S * V * 8
    out["cfg3_retrieve_fuse"] = {"ms": fuse_ms, "gbs": fuse_bytes / fuse_ms / 1e6, "frac_hbm": fuse_bytes / fuse_ms / 1e6 / hbm_peak,
                                 "bytes": fuse_bytes}
    _, per, _ = time_launches(gather, 20, 3)
    gather_ms = statistics.mean(per)
    gather_bytes = live * mat_bytes + rows * S * top_k * mat_bytes   # reads of live slots + writes of every slot
    out["cfg3_gather"] = {"ms": gather_ms, "gbs": gather_bytes / gather_ms / 1e6,
                          "frac_hbm": gather_bytes / gather_ms / 1e6 / hbm_peak, "bytes": gather_bytes}
    out["cfg3_tokens_per_s_route_plus_fuse"] = CFG3["B"] * CFG3["T"] / ((out["cfg3_topk_route_ms"] + fuse_ms) * 1e-3)
    del archives, gathered
    # ---- config 5 slab: 256 of the 4096 rows, T=32768, d=128 ----
    c5 = CFG5_SLAB
    k, v, q = make_scan_inputs(c5["rows"], c5["T"], c5["K"], c5["V"], device, seed=5)
    o = torch.empty_like(v)
    m_in = torch.zeros(c5["rows"], c5["V"], c5["K"], device=device)
    m_out = torch.empty_like(m_in)

    def scan5(_):
        cabi.check(lib.grmx_chunk_scan_fwd(k.data_ptr(), v.data_ptr(), q.data_ptr(), m_in.data_ptr(), o.data_ptr(),
                                           m_out.data_ptr(), c5["rows"], c5["T"], c5["K"], c5["V"], c5["decay"],
                                           cabi.BF16, cabi.F32, cabi.PATH_AUTO, stream))

    _, per, _ = time_launches(scan5, 3, 1)
    ms = statistics.mean(per)
    nbytes = c5["rows"] * c5["T"] * (2 * (2 * c5["K"] + c5["V"]) + 2 * c5["V"])
    out["cfg5_slab_scan"] = {"rows": c5["rows"], "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm_peak,
                             "row_tokens_per_s": c5["rows"] * c5["T"] / (ms * 1e-3),
                             "tokens_per_s_at_16_heads": c5["rows"] / 16 * c5["T"] / (ms * 1e-3)}
    return out


def cpu_reference_step(sample_rows, seed=0):
    """One pass of the config-2 scan over `sample_rows` rows on the host: returns seconds."""
    import numpy as np

    import oracle

    rows, T, K, V, decay = sample_rows, CFG2["T"], CFG2["K"], CFG2["V"], CFG2["decay"]
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(rows, T, K, generator=g), dim=-1, eps=1e-6)
    k = torch.nn.functional.normalize(torch.randn(rows, T, K, generator=g), dim=-1, eps=1e-6)
    v = torch.randn(rows, T, V, generator=g)
    m = torch.zeros(rows, V, K)
    ref = oracle.reference_ops()
    if ref is not None:
        t0 = time.perf_counter()
        ref.chunk_update_forward(k, v, q, m, decay)
        return time.perf_counter() - t0, "reference"
    kn, vn, qn, mn = (np.ascontiguousarray(t.numpy()) for t in (k, v, q, m))
    t0 = time.perf_counter()
    oracle.c_chunk_update(kn, vn, qn, mn, decay)
    return time.perf_counter() - t0, "port"


def cpu_baseline(sample_rows, reps):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cpu_reference_step(min(sample_rows, 8))      # warm-up
    times, kind = [], "port"
    for _ in range(reps):
        dt, kind = cpu_reference_step(sample_rows)
        times.append(dt)
    dt = statistics.median(times)
    tokens = CFG2["B"] * CFG2["T"] * sample_rows / (CFG2["B"] * CFG2["Hd"])
    what = ("grm::chunk_update_forward, the reference's compiled CPU op (grm/csrc/grm_cuda.cpp:46-90)"
            if kind == "reference" else "C restatement of the sequential scan (oracle/grm_oracle.c)")
    return {"value": tokens / dt, "unit": "tokens/s", "cores": cores, "kind": kind,
            "sample": f"{sample_rows} of 64 (b,h) rows x T=2048, fp32, median of {reps}; {what}", "seconds": dt}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    rows = CFG2["B"] * CFG2["Hd"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_step(8)
    times, kind = [], "port"
    steps = max(1, min(args.steps, 5))
    for _ in range(steps):
        dt, kind = cpu_reference_step(rows)
        times.append(dt)
    total = sum(times)
    tokens = CFG2["B"] * CFG2["T"]
    value = tokens * steps / total
    return {
        "impl": "reference",
        "metric": "memory-path tokens/s",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": steps,
        "warmup": args.warmup,
        "ms_per_step": total / steps * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp32",
        "data": "synthetic",
        "config": {"workload": "chunked linear-memory update + query kernel alone: B=8 H=8 T=2048 d_k=64 d_v=64, "
                               "decay 0.97, zero start state (CPU, one batch)"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind,
                         "sample": f"all 64 (b,h) rows x T=2048 per step, fp32, {steps} steps"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", choices=["engine", "reference"], default="engine")
    parser.add_argument("--skip-extras", action="store_true",
                        help="main workload only: no CPU baseline, no other workloads (small footprint for profiling)")
    parser.add_argument("--with-workspace", action="store_true",
                        help="time the two-kernel variant of the cut (piece-state kernel + scan over a caller workspace)")
    parser.add_argument("--full-occupancy-only", action="store_true",
                        help="run only the one-row-per-SM scan of the extras and print its figures (for profiling)")
    parser.add_argument("--config4-only", action="store_true",
                        help="run only the config-4 language-model forward of the extras (for profiling)")
    parser.add_argument("--segment-retrieval-only", action="store_true",
                        help="run only the per-token routing and select-fuse kernels of one config-4 segment (for profiling)")
    args = parser.parse_args(argv)
    args.warmup = max(args.warmup, 3)

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
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    if args.full_occupancy_only:
        from rnn_with_grm_b200 import cabi
        print(json.dumps({"full_occupancy_scan": full_occupancy_scan(cabi.load(), device, load_peaks()[0])}), flush=True)
        return 0
    if args.config4_only:
        from rnn_with_grm_b200 import cuda_ops
        if not cuda_ops.load_grm_cuda_extension():
            raise RuntimeError("grm_cuda extension failed to load: " + cuda_ops.get_grm_cuda_runtime_status()["load_error"])
        print(json.dumps({"cfg4_model": config4_model(device)}), flush=True)
        return 0
    if args.segment_retrieval_only:
        from rnn_with_grm_b200 import cabi
        print(json.dumps({"cfg4_segment_retrieval": segment_retrieval(cabi.load(), device, load_peaks()[0], launches=4)}),
              flush=True)
        return 0
    try:
        result = run_engine(args, rank, world, device)
        if result is not None:
            print(json.dumps(result), flush=True)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
