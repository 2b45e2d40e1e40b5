#!/usr/bin/env python
"""Benchmark of the fused Softmax + TopK hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default `llm_vocab_f32`): fp32 logits [64, 128256] ~ N(0,1) with 20
spikes per row, temperature 0.8, k = 50 -- the configuration the headline
metric is quoted on.  One step = one pass of the fused operator over one batch.
With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank
processes its own batch of rows: rows shard across GPUs with no collective on
the data path, so scaling is weak and `value` is N * rows / step time.

Timing: W warm-up steps, then exactly K steps between CUDA events on the
launching stream, bracketed by a barrier and a device synchronize; the maximum
over ranks is reported.  Consecutive steps read different input buffers (8
buffers, 263 MB in total, more than the 126 MB L2), so every step streams its
logits from HBM.

The JSON line carries, besides the contract keys:
  roofline      algorithmic bytes per launch / mean launch duration, against the
                measured HBM copy bandwidth of this pool
  e2e           same metric through host buffers: pinned host logits -> device,
                the operator, results -> host, every step
  cpu_baseline  the CPU oracle (a port of the reference's own CPU statement of
                this path) timed on this machine's cores (rank 0, N = 1 only)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (rows, cols, dtype, k, inv_temperature)
    "llm_vocab_f32": (64, 128256, torch.float32, 50, 1.25),
    "llm_vocab_f16": (64, 128256, torch.float16, 50, 1.25),
    "batched_classifier": (256, 1000, torch.float32, 5, 1.0),
    "sharded_vocab_bf16": (512, 256000, torch.bfloat16, 64, 1.0),
}
NBUF = 8
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the streaming kernel, from the ncu
# capture summarised in profiles/softmax_topk_stream_llm_vocab_f32_full.md; None for workloads
# without a capture.
NCU_TRAFFIC_BYTES = {"llm_vocab_f32": 32997376}


def algorithmic_bytes(rows, cols, dtype, k):
    esz = torch.empty((), dtype=dtype).element_size()
    return rows * cols * esz + rows * k * (esz + 4)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.001):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML not reachable: report that instead of clocks
            self.nv = None
        self.period = period_s

    def _one(self):
        nv = self.nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
        r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
            else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        for n, bit in names.items():
            if r & bit:
                self.reasons.add(n)

    def _run(self):
        while not self._stop.is_set():
            try:
                self._one()
            except Exception:
                break
            time.sleep(self.period)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def sample_now(self):
        if self.nv:
            try:
                self._one()
            except Exception:
                pass

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        if self.nv and not self.samples:
            try:
                self._one()
            except Exception:
                pass

    def summary(self):
        if not self.nv or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml_unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_inputs(name, seed_base, device):
    from vkop_b200 import workloads

    rows, cols, dtype, k, inv_t = WORKLOADS[name]
    bufs = []
    for b in range(NBUF):
        if name.startswith("llm_vocab"):
            x = workloads.llm_vocab(seed=seed_base + b, rows=rows, cols=cols, dtype=dtype)
        elif name == "batched_classifier":
            x = workloads.batched_classifier(seed=seed_base + b, rows=rows, cols=cols)
        else:
            x = workloads.spiked_normal(rows, cols, 32, 9.0, 1.5, seed_base + b, dtype)
        bufs.append(x)
    return bufs


def run_reference(args, rank, world):
    """The reference's CPU statement of the path (oracle port), all host threads, on the same workload."""
    if rank != 0:
        return
    import oracle
    from tests.util import ORACLE_DTYPE, to_oracle_array
    from vkop_b200 import workloads

    rows, cols, dtype, k, inv_t = WORKLOADS[args.workload]
    x = make_inputs(args.workload, 1000, "cpu")[0]
    xa = to_oracle_array(x)
    # every host thread, whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to 1)
    oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    cores = oracle.num_threads()

    def step():
        oracle.softmax_topk(xa, k, inv_t, dtype=ORACLE_DTYPE[dtype], sum_mode=oracle.SUM_F32_SEQUENTIAL, full_sort=True)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = rows / dt
    line = {
        "impl": "reference", "metric": "fused_softmax_topk_rows_per_s", "value": value, "unit": "rows/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": str(dtype).replace("torch.", ""),
        "data": "synthetic",
        "config": {"workload": args.workload, "rows": rows, "cols": cols, "k": k, "inv_temperature": inv_t},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": "port",
                         "sample": f"one batch of {rows} rows per step; max -> exp -> sequential fp32 sum -> divide -> "
                                   "full sort, as core/function.cpp:150-183, OpenMP over rows"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_nms(args, local_rank):
    """Side line, not the headline metric: the NMS operator on the YOLO-style detect configuration
    (16 images x 80 classes x 8400 anchors, threshold 0.25, per-class top-300, IoU 0.45, 300 kept)."""
    from vkop_b200 import capi, workloads

    torch.cuda.set_device(local_rank)
    sets = []
    for b in range(4):  # 4 x 45 MB of scores and boxes rotate: more than the L2 holds
        boxes, scores = workloads.yolo_detect(seed=3 + b)
        sets.append((boxes.cuda(), scores.cuda()))
    B, Cn, N = sets[0][1].shape
    cap = B * Cn * 300
    rows = torch.empty((cap, 3), dtype=torch.int32, device="cuda")
    count = torch.empty(1, dtype=torch.int32, device="cuda")
    ws = None
    steps = min(args.steps, 200)

    def step(i):
        nonlocal ws
        bx, sc = sets[i % len(sets)]
        if ws is None:
            d = capi.NmsDesc(num_batch=B, num_class=Cn, num_boxes=N, capacity_rows=cap, **workloads.YOLO_PARAMS)
            ws = capi.Workspace(capi.nms_workspace_bytes(d), bx.device)
        capi.nms(bx, sc, capacity_rows=cap, workspace=ws, out=(rows, count), **workloads.YOLO_PARAMS)

    n0 = capi.launch_count()
    step(0)
    per_step = capi.launch_count() - n0
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    peak, peak_kind = measured_peak()
    nbytes = B * Cn * N * 4 + B * N * 16
    print(json.dumps({
        "metric": "nms_images_per_s", "value": B / (ms * 1e-3), "unit": "images/s", "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "float32", "data": "synthetic",
        "config": {"workload": "yolo_nms", "images": B, "classes": Cn, "anchors": N, "kept_rows": int(count.item()),
                   "us_per_class_problem": ms * 1e3 / (B * Cn), "l2": "4 input sets (180 MB) rotate > L2"},
        "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                     "note": "score scan only; the suppression sweep is latency-bound"},
        "gpu_launches": per_step * steps}))


def run_vocab_sharded(args, rank, local_rank, world):
    """Side line: one batch whose columns are split over the ranks (strong scaling).  A step = partial
    selection on the local column slice, all-gather of the per-row packets (NCCL), merge on every rank."""
    import torch.distributed as dist

    from vkop_b200 import sharded, workloads

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rows, cols, dtype, k, inv_t = WORKLOADS[args.workload]
    lo, hi = sharded.split_even(cols, world, rank)
    # every rank draws its own slice (the values of a slice do not depend on the others)
    slices = [workloads.spiked_normal(rows, hi - lo, max(1, 32 // world), 9.0, 1.5, 7000 + 100 * rank + b, dtype).to(dev)
              for b in range(NBUF)]
    op = sharded.VocabShardedSoftmaxTopk(rows, hi - lo, lo, k, dtype, inv_t, device=dev, exchange=args.exchange)
    steps = min(args.steps, 500)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        op(slices[i % NBUF])
    barrier()
    # Launched from the host, step by step: capturing the NCCL collective into a CUDA graph hung a
    # two-rank run on this pool (most likely the process group's watchdog thread touching CUDA during
    # the capture), so no graph here.
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        op(slices[i % NBUF])
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    peak, peak_kind = measured_peak()
    esz = slices[0].element_size()
    nbytes = rows * cols * esz + rows * k * (esz + 4)
    if rank == 0:
        print(json.dumps({
            "metric": "fused_softmax_topk_rows_per_s", "value": rows / (ms * 1e-3), "unit": "rows/s", "n_gpus": world,
            "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": str(dtype).replace("torch.", ""), "data": "synthetic",
            "config": {"workload": args.workload, "rows": rows, "cols": cols, "cols_per_gpu": hi - lo, "k": k,
                       "sharding": f"vocab x{world}", "exchange": ("NCCL all-gather of per-row packets" if args.exchange == "nccl" or world == 1
                                    else "stores into peer memory + flags (NVLink)") + " + merge kernel",
                       "launch": "host",
                       "packet_bytes_per_rank": rows * (4 + 2 * k) * 4,
                       "l2": f"inputs rotate over {NBUF} buffers ({NBUF * rows * (hi - lo) * esz >> 20} MiB per rank)"},
            "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peak * world, "unit": "GB/s",
                         "frac": nbytes / (ms * 1e-3) / 1e9 / (peak * world), "traffic": None, "peak_kind": peak_kind}}))
    if world > 1:
        if op.peer is not None:
            dist.barrier()
            op.peer.close()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llm_vocab_f32", choices=sorted(WORKLOADS) + ["yolo_nms"])
    ap.add_argument("--splits", type=int, default=0, help="chunks per row (0 = automatic)")
    ap.add_argument("--path", default="auto", choices=["auto", "chunk", "stream", "radix", "bulk"])
    ap.add_argument("--serialize", action="store_true",
                    help="do not declare the resident inputs ready: every launch fully waits for the one before")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of replaying a CUDA graph")
    ap.add_argument("--sharding", default="rows", choices=["rows", "vocab"],
                    help="N > 1: rows = every rank its own batch (weak scaling, no collective); vocab = the columns of "
                         "one batch split over the ranks, packets all-gathered and merged (strong scaling)")
    ap.add_argument("--exchange", default="nccl", choices=["nccl", "peer"],
                    help="--sharding vocab: how the packets travel (NCCL all-gather, or stores into peer memory)")
    ap.add_argument("--graph-steps", type=int, default=256, help="steps captured in the CUDA graph that is replayed")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        args.steps = 5 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
        run_reference(args, rank, world)
        return
    args.steps = 2048 if args.steps is None else args.steps
    args.warmup = 20 if args.warmup is None else args.warmup
    if args.workload == "yolo_nms":
        run_nms(args, local_rank)
        return
    if args.sharding == "vocab":
        run_vocab_sharded(args, rank, local_rank, world)
        return

    from vkop_b200 import capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    rows, cols, dtype, k, inv_t = WORKLOADS[args.workload]
    host = make_inputs(args.workload, 1000 + 100 * rank, "cpu")
    bufs = [h.to(dev) for h in host]
    values = torch.empty((rows, k), dtype=dtype, device=dev)
    indices = torch.empty((rows, k), dtype=torch.int32, device=dev)
    path = {"auto": capi.PATH_AUTO, "chunk": capi.PATH_CHUNK, "stream": capi.PATH_STREAM, "radix": capi.PATH_RADIX, "bulk": capi.PATH_BULK}[args.path]
    # the inputs of every step are resident and complete before the timed region starts
    flags = 0 if args.serialize else capi.FLAG_INPUT_READY
    desc = capi.make_desc(bufs[0], k, inv_t, splits=args.splits, path=path, flags=flags)
    ws = capi.Workspace(capi.softmax_topk_workspace_bytes(desc), dev)

    import ctypes as C

    L = capi.lib()
    dref = C.byref(desc)
    in_ptrs = [b.data_ptr() for b in bufs]
    vptr, iptr, wsptr, wsbytes = values.data_ptr(), indices.data_ptr(), ws.ptr, ws.buf.numel()

    def step(i, stream):
        rc = L.vkop_cuda_softmax_topk(dref, in_ptrs[i % NBUF], vptr, iptr, wsptr, wsbytes, stream)
        if rc != 0:
            raise capi.VkopError(rc, "softmax_topk")

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream().cuda_stream
    n0 = capi.launch_count()
    step(0, stream)
    launches_per_step = capi.launch_count() - n0
    for i in range(max(args.warmup, 3)):
        step(i, stream)
    barrier()
    graph = None
    gsteps = max(NBUF, (args.graph_steps // NBUF) * NBUF)
    if not args.no_graph and args.steps >= gsteps:
        # the launch-bound loop is captured once (consecutive steps read different buffers) and replayed
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            cs = torch.cuda.current_stream().cuda_stream
            for i in range(gsteps):
                step(i, cs)
        for _ in range(3):
            graph.replay()
        barrier()
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    e0.record()
    done = 0
    if graph is not None:
        for _ in range(args.steps // gsteps):
            graph.replay()
        done = (args.steps // gsteps) * gsteps
    for i in range(done, args.steps):
        step(i, stream)
    e1.record()
    sampler.sample_now()  # the queued steps are still running: one sample even when the region is shorter than a period
    barrier()
    sampler.stop()
    launches = launches_per_step * args.steps
    ms = e0.elapsed_time(e1) / args.steps
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())

    # ---- end to end: pinned host logits -> device -> operator -> results to host, every step ----
    e2e = None
    if not args.no_e2e:
        # the reference-facing call: the C++ Runtime mirror with Softmax + TopK registered as
        # post-processing (what the reference's benchmark program builds), fed HOST buffers
        from vkop_b200 import host_api

        pinned = [h.pin_memory() for h in host[:2]]
        hv = torch.empty((rows, k), dtype=dtype).pin_memory()
        hi = torch.empty((rows, k), dtype=torch.int32).pin_memory()
        pipe = host_api.HostPipeline(dev.index or 0, rows, cols, capi._TORCH_DTYPE[dtype], k, 1.0 / inv_t, fuse=True)
        e2e_steps = max(3, min(args.steps, 50))
        pin_ptrs = [p_.data_ptr() for p_ in pinned]

        def e2e_step(i):
            # logits host -> device, the fused operator, k values and indices of every row back to the host
            pipe.run_ptr(pin_ptrs[i % 2], hv.data_ptr(), hi.data_ptr())

        for i in range(3):
            e2e_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        esz = bufs[0].element_size()
        e2e = {"value": rows * world / (float(t.item()) * 1e-3), "unit": "rows/s",
               "h2d_bytes_per_step": rows * cols * esz, "d2h_bytes_per_step": rows * k * (esz + 4),
               "steps": e2e_steps, "ms_per_step": float(t.item()),
               "api": "vkop_host_pipeline_run (C++ Runtime::RegisterPostProcess Softmax+TopK, host buffers)"}

    # ---- parity spot check of the last step against the oracle (outside every timed region) ----
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        from tests.util import ORACLE_DTYPE, to_oracle_array

        xa = to_oracle_array(host[0])
        oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
        # parity spot check: one more step on buffer 0, indices against the oracle, bit for bit
        step(0, stream)
        torch.cuda.synchronize()
        _, want_idx = oracle.softmax_topk(xa, k, inv_t, dtype=ORACLE_DTYPE[dtype])
        if not (indices.cpu().numpy() == want_idx).all():
            raise SystemExit("bench.py: the GPU result differs from the oracle")
        reps, t0 = 0, time.perf_counter()
        while reps < 10 or time.perf_counter() - t0 < 2.0:  # a bounded sample: about 2 s on all cores
            oracle.softmax_topk(xa, k, inv_t, dtype=ORACLE_DTYPE[dtype], sum_mode=oracle.SUM_F32_SEQUENTIAL,
                                full_sort=True)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        cpu_baseline = {"value": rows / dt, "unit": "rows/s", "cores": oracle.num_threads(), "kind": "port",
                        "sample": f"{reps} passes over one batch of {rows} rows ({dt * reps:.1f} s wall): max -> exp -> "
                                  "sequential fp32 sum -> divide -> full sort (core/function.cpp:150-183), "
                                  "OpenMP over rows"}

    if rank == 0:
        peak, peak_kind = measured_peak()
        abytes = algorithmic_bytes(rows, cols, dtype, k)
        achieved = abytes / (ms_max * 1e-3) / 1e9
        line = {
            "metric": "fused_softmax_topk_rows_per_s", "value": rows * world / (ms_max * 1e-3), "unit": "rows/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_max,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": str(dtype).replace("torch.", ""), "data": "synthetic",
            "config": {"workload": args.workload, "rows_per_gpu": rows, "cols": cols, "k": k, "inv_temperature": inv_t,
                       "sharding": f"rows x{world}" if world > 1 else "none",
                       "l2": f"inputs rotate over {NBUF} buffers ({NBUF * rows * cols * bufs[0].element_size() >> 20} MiB) > L2",
                       "path": args.path, "input_ready_flag": not args.serialize, "launch": "host" if graph is None else f"cuda graph of {gsteps} steps"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": abytes, "pct_of_8TBs": achieved / 8000.0 * 100.0},
            "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
