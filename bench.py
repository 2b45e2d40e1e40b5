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

The steps are captured once in a CUDA graph (K steps when K <= 256, else 256 that are replayed),
the graph is replayed untimed as extra warm-up, and the timed region replays it: the launch-bound
loop then costs no host time.  `--no-graph` launches every step from the host instead.

The JSON line carries, besides the contract keys:
  roofline      algorithmic bytes per launch / mean launch duration, against the
                measured HBM copy bandwidth of this pool
  e2e           same metric through host buffers: pinned host logits -> device,
                the operator, results -> host, every step
  serialized    the same steps without VKOP_FLAG_INPUT_READY: every call waits for the one before
  vocab_sharded the 512 x 256000 bf16, k = 64 configuration with the columns split over the N ranks
                (partial selection per rank, packet exchange, merge); at N = 1 the whole matrix on one GPU
  cpu_baseline  the reference's own CPU code for this path (core/function.cpp, compiled into oracle/_ref)
                or, where that is not built, the oracle port of it, timed on this machine's cores
                (rank 0, N = 1 only), with torch-CPU softmax + topk beside it
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
    "long_row": (1, 16777216, torch.float32, 1024, 1.0),  # one row of 16 Mi logits, k = 1024: the radix-select path
}
NBUF = 8
GATE_CYCLES = 600_000  # about 0.3 ms of device spin in front of a timed region (see timed())
FALLBACK_HBM_GBS = 6650.0
# ncu capture summaries that state the DRAM traffic of one launch of the workload's dominant kernel
TRAFFIC_SUMMARY = {"llm_vocab_f32": "softmax_topk_stream_llm_vocab_f32_full.md"}


def ncu_traffic_bytes(workload):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch, read from the committed capture summary
    (None for workloads without one)."""
    import re

    name = TRAFFIC_SUMMARY.get(workload)
    path = os.path.join(ROOT, "profiles", name) if name else None
    if not path or not os.path.exists(path):
        return None
    total = 0
    with open(path) as f:
        for line in f:
            m = re.match(r"\|\s*`dram__bytes_(read|write)\.sum`\s*\|\s*([0-9 ]+)\s*B", line)
            if m:
                total += int(m.group(2).replace(" ", ""))
    return total or None


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
        elif name == "long_row":
            x = workloads.long_row(seed=seed_base + b, cols=cols)
        else:
            x = workloads.spiked_normal(rows, cols, 32, 9.0, 1.5, seed_base + b, dtype)
        bufs.append(x)
    return bufs


def cpu_reference_step(name):
    """One CPU pass over one batch of the workload with every host thread.  Returns (step function, cores, kind,
    what it runs): the reference's own Function::get_top_k_predictions compiled from its source (oracle/_ref;
    fp32 only) when that library exists, else the oracle port of it."""
    import oracle
    from oracle import ref

    rows, cols, dtype, k, inv_t = WORKLOADS[name]
    x = make_inputs(name, 1000, "cpu")[0]
    ncores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if dtype == torch.float32 and ref.available():
        xa = x.numpy()
        ref.set_num_threads(ncores)
        return (lambda: ref.function_top_k_predictions(xa, k, inv_t)), ncores, "reference", \
            "core/function.cpp Function::get_top_k_predictions (max, exp, sequential fp32 sum, divide, std::sort), " \
            "compiled from the reference source, one call per row, OpenMP over rows"
    xa = oracle.to_oracle_array(x)
    # every host thread, whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to 1)
    oracle.set_num_threads(ncores)
    dt = oracle.oracle_dtype(dtype)
    return (lambda: oracle.softmax_topk(xa, k, inv_t, dtype=dt, sum_mode=oracle.SUM_F32_SEQUENTIAL, full_sort=True)), \
        oracle.num_threads(), "port", \
        "oracle port of core/function.cpp:150-183 (max, exp, sequential fp32 sum, divide, full sort; qsort where the " \
        "reference uses std::sort), OpenMP over rows"


def run_reference(args, rank, world):
    """The reference's CPU statement of the path, all host threads, on the same workload."""
    if rank != 0:
        return
    rows, cols, dtype, k, inv_t = WORKLOADS[args.workload]
    step, cores, kind, what = cpu_reference_step(args.workload)
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
        "config": {"workload": args.workload, "rows_per_gpu": rows, "cols": cols, "k": k, "inv_temperature": inv_t},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": kind,
                         "sample": f"one batch of {rows} rows per step; " + what},
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

    # end to end: scores and boxes start in pinned host memory, the kept rows and their count come back
    host = [(bx.cpu().pin_memory(), sc.cpu().pin_memory()) for bx, sc in sets]
    out_rows = torch.empty((cap, 3), dtype=torch.int32).pin_memory()
    out_count = torch.empty(1, dtype=torch.int32).pin_memory()
    dbx, dsc = torch.empty_like(sets[0][0]), torch.empty_like(sets[0][1])

    def e2e_step(i):
        hb, hs = host[i % len(host)]
        dbx.copy_(hb, non_blocking=True)
        dsc.copy_(hs, non_blocking=True)
        capi.nms(dbx, dsc, capacity_rows=cap, workspace=ws, out=(rows, count), **workloads.YOLO_PARAMS)
        out_count.copy_(count, non_blocking=True)
        out_rows.copy_(rows, non_blocking=True)
        torch.cuda.synchronize()

    e2e_steps = min(steps, 20)
    for i in range(3):
        e2e_step(i)
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3

    # CPU baseline: the oracle's port of shaders/nms.comp (greedy sweep per (image, class), OpenMP over the
    # problems) on the same 16 images, every host thread
    import oracle
    ncores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.set_num_threads(ncores)
    hb, hs = host[0][0].numpy(), host[0][1].numpy()
    oracle.nms(hb, hs, **workloads.YOLO_PARAMS)
    t0 = time.perf_counter()
    cpu_reps = 3
    for _ in range(cpu_reps):
        oracle.nms(hb, hs, **workloads.YOLO_PARAMS)
    cpu_s = (time.perf_counter() - t0) / cpu_reps
    print(json.dumps({
        "metric": "nms_images_per_s", "value": B / (ms * 1e-3), "unit": "images/s", "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "float32", "data": "synthetic",
        "config": {"workload": "yolo_nms", "images": B, "classes": Cn, "anchors": N, "kept_rows": int(count.item()),
                   "us_per_class_problem": ms * 1e3 / (B * Cn), "l2": "4 input sets (180 MB) rotate > L2"},
        "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                     "note": "score scan only; the kernel is bound by instruction issue (IoU mask), not by HBM"},
        "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "images/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": cap * 12 + 4},
        "cpu_baseline": {"value": B / cpu_s, "unit": "images/s", "cores": oracle.num_threads(), "kind": "port",
                         "sample": "the same 16 images, %d passes of the oracle's port of shaders/nms.comp" % cpu_reps},
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
                                    else "stores into peer memory + flags (NVLink)" + (", C++ operator" if args.exchange == "native" else "")) + " + merge kernel",
                       "launch": "host",
                       "packet_bytes_per_rank": rows * (4 + 2 * k) * 4,
                       "l2": f"inputs rotate over {NBUF} buffers ({NBUF * rows * (hi - lo) * esz >> 20} MiB per rank)"},
            "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peak * world, "unit": "GB/s",
                         "frac": nbytes / (ms * 1e-3) / 1e9 / (peak * world), "traffic": None, "peak_kind": peak_kind}}))
    if world > 1:
        if op.peer is not None or op.native is not None:
            dist.barrier()
            op.close()
        dist.destroy_process_group()


def measure_vocab_sharded(args, rank, world, dev, dist, barrier, max_over_ranks):
    """The vocabulary-sharded configuration (512 x 256000 bf16, k = 64) as a sub-measurement of the default run:
    the columns are split evenly over the `world` ranks; a step = partial selection on the local slice, packet
    exchange (stores into peer memory, or an NCCL all-gather), merge on every rank.  At one GPU the whole matrix
    is selected on that GPU (no exchange): that time is the T1 of the parallel efficiency T1 / (N * TN)."""
    from vkop_b200 import sharded, workloads

    name = "sharded_vocab_bf16"
    rows, cols, dtype, k, inv_t = WORKLOADS[name]
    lo, hi = sharded.split_even(cols, world, rank)
    nbuf = 4  # 4 x 262 MB / N per rank: more than the L2 holds at every N up to 8
    # every rank draws its own slice (the values of a slice do not depend on the others)
    slices = [workloads.spiked_normal(rows, hi - lo, max(1, 32 // world), 9.0, 1.5, 7000 + 100 * rank + b, dtype).to(dev)
              for b in range(nbuf)]
    exchange = "none" if world == 1 else args.exchange
    # one GPU: the C++ operator too (partial + merge, no exchange)
    want = "native" if (world == 1 and args.exchange == "native") else ("nccl" if world == 1 else args.exchange)
    try:
        op = sharded.VocabShardedSoftmaxTopk(rows, hi - lo, lo, k, dtype, inv_t, device=dev, exchange=want)
    except Exception as e:  # peer mapping refused (no peer access between these GPUs): the all-gather still works
        if want == "nccl" or world == 1:
            raise
        exchange = f"nccl ({want} exchange unavailable: {type(e).__name__})"
        op = sharded.VocabShardedSoftmaxTopk(rows, hi - lo, lo, k, dtype, inv_t, device=dev, exchange="nccl")
    steps = max(5, min(args.steps, 100))
    for i in range(max(args.warmup, 3)):
        op(slices[i % nbuf])
    barrier()
    # launched from the host, step by step (a collective is not captured into a graph here)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        op(slices[i % nbuf])
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1) / steps)
    timed_out = op.timed_out()
    if op.peer is not None or op.native is not None:
        barrier()
        op.close()
    if timed_out:
        raise SystemExit("bench.py: a bounded wait for the peers' packets gave up")
    esz = slices[0].element_size()
    nbytes = rows * cols * esz + rows * k * (esz + 4)
    peak, peak_kind = measured_peak()
    return {"workload": name, "rows": rows, "cols": cols, "cols_per_gpu": hi - lo, "k": k, "n_gpus": world,
            "ms_per_step": ms, "steps": steps, "value": rows / (ms * 1e-3), "unit": "rows/s", "scaling": "strong",
            "exchange": {"none": "none (one GPU holds every column)", "peer": "stores into peer memory + flags (NVLink), then the merge kernel",
                         "native": "stores into peer memory + flags (NVLink), then the merge kernel; the step is one call of the C++ operator ops::SoftmaxTopkSharded",
                         "nccl": "NCCL all-gather of per-row packets, then the merge kernel"}.get(exchange, exchange),
            "launch": "host", "packet_bytes_per_rank": rows * (4 + 2 * k) * 4,
            "hbm_frac_of_n_gpus": nbytes / (ms * 1e-3) / 1e9 / (peak * world), "peak_kind": peak_kind,
            "efficiency": "T1 / (N * TN) with T1 = ms_per_step of the one-GPU run of this same sub-measurement"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-gate", action="store_true",
                    help="do not enqueue the short device spin in front of the timed region (the host's launch latency then counts)")
    ap.add_argument("--workload", default="llm_vocab_f32", choices=sorted(WORKLOADS) + ["yolo_nms"])
    ap.add_argument("--splits", type=int, default=0, help="chunks per row (0 = automatic)")
    ap.add_argument("--path", default="auto", choices=["auto", "chunk", "stream", "radix", "bulk"])
    ap.add_argument("--serialize", action="store_true",
                    help="do not declare the resident inputs ready: every launch fully waits for the one before")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-serialized", action="store_true", help="skip the second loop without VKOP_FLAG_INPUT_READY")
    ap.add_argument("--no-vocab-sharded", action="store_true", help="skip the vocabulary-sharded sub-measurement")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of replaying a CUDA graph")
    ap.add_argument("--sharding", default="rows", choices=["rows", "vocab"],
                    help="N > 1: rows = every rank its own batch (weak scaling, no collective); vocab = the columns of "
                         "one batch split over the ranks, packets all-gathered and merged (strong scaling)")
    ap.add_argument("--exchange", default="native", choices=["nccl", "peer", "native"],
                    help="vocabulary sharding: how the packets travel (native: stores into peer memory, the whole step owned by "
                         "the C++ operator ops::SoftmaxTopkSharded; peer: the same exchange orchestrated from Python; nccl: an "
                         "NCCL all-gather)")
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
    if args.steps < 1:
        raise SystemExit("--steps must be at least 1")
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

    rows, cols, dtype, k, inv_t = WORKLOADS[args.workload]
    host = make_inputs(args.workload, 1000 + 100 * rank, "cpu")
    bufs = [h.to(dev) for h in host]
    values = torch.empty((rows, k), dtype=dtype, device=dev)
    indices = torch.empty((rows, k), dtype=torch.int32, device=dev)
    path = {"auto": capi.PATH_AUTO, "chunk": capi.PATH_CHUNK, "stream": capi.PATH_STREAM, "radix": capi.PATH_RADIX, "bulk": capi.PATH_BULK}[args.path]

    import ctypes as C

    L = capi.lib()
    in_ptrs = [b.data_ptr() for b in bufs]
    vptr, iptr = values.data_ptr(), indices.data_ptr()

    class Loop:
        """K steps of the operator with one descriptor (its own workspace), captured in a CUDA graph."""

        def __init__(self, flags):
            self.desc = capi.make_desc(bufs[0], k, inv_t, splits=args.splits, path=path, flags=flags)
            self.ws = capi.Workspace(capi.softmax_topk_workspace_bytes(self.desc), dev)
            self.graph, self.gsteps = None, 0

        def step(self, i, stream):
            rc = L.vkop_cuda_softmax_topk(C.byref(self.desc), in_ptrs[i % NBUF], vptr, iptr, self.ws.ptr, self.ws.buf.numel(), stream)
            if rc != 0:
                raise capi.VkopError(rc, "softmax_topk")

        def prepare(self, steps, warmup):
            stream = torch.cuda.current_stream().cuda_stream
            for i in range(max(warmup, 3)):
                self.step(i, stream)
            torch.cuda.synchronize()
            if not args.no_graph:
                # the launch-bound loop is captured once (consecutive steps read different buffers) and replayed
                self.gsteps = steps if steps <= args.graph_steps else max(NBUF, (args.graph_steps // NBUF) * NBUF)
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
                    cs = torch.cuda.current_stream().cuda_stream
                    for i in range(self.gsteps):
                        self.step(i, cs)
                for _ in range(2):  # untimed: more warm-up than asked for
                    self.graph.replay()
                torch.cuda.synchronize()

        def run(self, steps):
            """Enqueues exactly `steps` steps."""
            stream = torch.cuda.current_stream().cuda_stream
            done = 0
            if self.graph is not None:
                for _ in range(steps // self.gsteps):
                    self.graph.replay()
                done = (steps // self.gsteps) * self.gsteps
            for i in range(done, steps):
                self.step(i, stream)

    # the inputs of every step are resident and complete before the timed region starts: the main
    # loop says so (VKOP_FLAG_INPUT_READY); the second loop leaves the flag clear (every call waits)
    n0 = capi.launch_count()
    main = Loop(0 if args.serialize else capi.FLAG_INPUT_READY)
    main.step(0, torch.cuda.current_stream().cuda_stream)
    launches_per_step = capi.launch_count() - n0
    main.prepare(args.steps, args.warmup)
    waiting = None
    if not args.serialize and not args.no_serialized:
        waiting = Loop(0)
        waiting.prepare(args.steps, args.warmup)

    # graphs are captured before the process group exists (its watchdog thread must not meet a capture)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(loop, steps, sampler=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.start()
        # a short spin is enqueued first, so that the host has every step queued before the device reaches the
        # first event: the region then holds K steps of device work and none of the host's launch latency
        # (about 50 us for one graph launch on an idle device, a quarter of a 20-step region)
        if not args.no_gate:
            torch.cuda._sleep(GATE_CYCLES)
        e0.record()
        loop.run(steps)
        e1.record()
        if sampler:
            sampler.sample_now()  # the queued steps are still running: one sample even when the region is shorter than a period
        barrier()
        if sampler:
            sampler.stop()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    sampler = ClockSampler(local_rank)
    ms_max = timed(main, args.steps, sampler)
    launches = launches_per_step * args.steps
    graph = main.graph
    gsteps = main.gsteps
    serialized = None
    if waiting is not None:
        ms_w = timed(waiting, args.steps)
        serialized = {"ms_per_step": ms_w, "value": rows * world / (ms_w * 1e-3), "unit": "rows/s",
                      "input_ready_flag": False, "ratio_to_overlapping": ms_w / ms_max}

    vocab_sharded = None
    if not args.no_vocab_sharded and args.workload == "llm_vocab_f32":
        vocab_sharded = measure_vocab_sharded(args, rank, world, dev, dist, barrier, max_over_ranks)

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
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / e2e_steps)
        esz = bufs[0].element_size()
        e2e = {"value": rows * world / (e2e_ms * 1e-3), "unit": "rows/s",
               "h2d_bytes_per_step": rows * cols * esz, "d2h_bytes_per_step": rows * k * (esz + 4),
               "steps": e2e_steps, "ms_per_step": e2e_ms,
               "api": "vkop_host_pipeline_run (C++ Runtime::RegisterPostProcess Softmax+TopK, host buffers)"}

    # ---- parity spot check of one more step against the oracle (outside every timed region), then
    # the CPU baselines on a bounded sample ----
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle

        xa = oracle.to_oracle_array(host[0])
        main.step(0, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        _, want_idx = oracle.softmax_topk(xa, k, inv_t, dtype=oracle.oracle_dtype(dtype))
        if not (indices.cpu().numpy() == want_idx).all():
            raise SystemExit("bench.py: the GPU result differs from the oracle")
        step_cpu, cores, kind, what = cpu_reference_step(args.workload)
        reps, t0 = 0, time.perf_counter()
        while reps < 10 or time.perf_counter() - t0 < 2.0:  # a bounded sample: about 2 s on all cores
            step_cpu()
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        cpu_baseline = {"value": rows / dt, "unit": "rows/s", "cores": cores, "kind": kind,
                        "sample": f"{reps} passes over one batch of {rows} rows ({dt * reps:.1f} s wall): " + what}
        # torch-CPU softmax + topk, the oracle the reference's own tests use (tests/TopkTest.cpp:73, tests/SoftmaxTest.cpp:138)
        torch.set_num_threads(cores)
        xt = host[0].float()
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or time.perf_counter() - t0 < 2.0:
            torch.topk(torch.softmax(xt * inv_t, dim=1), k, dim=1)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        cpu_baseline["torch_cpu"] = {"value": rows / dt, "unit": "rows/s", "cores": cores,
                                     "sample": f"{reps} passes of torch.softmax + torch.topk on one batch, {torch.get_num_threads()} threads"}

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
                       "path": args.path, "input_ready_flag": not args.serialize, "launch": "host" if graph is None else f"cuda graph of {gsteps} steps",
                       "timed_region": "CUDA events around the K steps" + ("" if args.no_gate else
                                       ", enqueued behind a 0.3 ms device spin so that the host's launch latency is outside")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": ncu_traffic_bytes(args.workload), "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": abytes, "pct_of_8TBs": achieved / 8000.0 * 100.0},
            "serialized": serialized, "vocab_sharded": vocab_sharded,
            "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
