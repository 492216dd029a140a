#!/usr/bin/env python
"""Benchmark of the hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step is one pass of one operator over one batch of seeded synthetic input.  The default
workload is the fp16 GEMM 4096^3 (the single-GPU configuration the headline metric is quoted
on); `--workload` selects any of the five configurations in heron_b200/workloads.py.

With N > 1 (launched under torch.distributed.run, one rank per GPU):
  * the GEMM configurations do not shard: every rank runs an independent replica ("weak");
  * the batched GEMM and the conv configurations split their batch / image dimension over the
    ranks with no data-path collective ("strong": total work fixed).

Rank 0 prints ONE JSON line.  `--impl reference` times the CPU port of the reference's x86
structure (oracle/dlboost_baseline.c) on the host cores instead; it is the only path in this
file that executes anything under oracle/ besides the cpu_baseline leg.
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

METRIC = "per-op TFLOPS/TOPS & % of B200 dense peak at 1/2/4/8 GPUs"
DEFAULT_WORKLOAD = "cfg2_gemm_f16_4096"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/; None where no capture has been taken.
NCU_TRAFFIC_BYTES = {
    "cfg2_gemm_f16_4096": 125e6,
    "cfg4_bmm_s8_attention": 155.3e6,
    "cfg3_conv_f16_resnet_s2": 12.9e6,
    "cfg5_conv_u8s8_resnet_s4": 74.8e6,
    "cfg1_gemm_u8s8_64": None,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


def arithmetic_dtype(cfg):
    return {"float16": "f16 (fp32 accumulate)", "int8": "s8 (s32 accumulate)",
            "uint8": "u8 x s8 (s32 accumulate)"}[cfg["in_dtype"]]


# ---- clocks -------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons of one GPU through NVML (read-only) while the
    timed region runs."""

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples = []
        self._stop_flag = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._stop_flag.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                self.samples.append((time.perf_counter(), mhz, reasons, watts))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_flag.set()

    def summary(self, t0, t1):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        nv = self.nv
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or \
            [min(self.samples, key=lambda s: abs(s[0] - 0.5 * (t0 + t1)))]
        mhz = sorted(s[1] for s in inside)
        bits = 0
        for s in inside:
            bits |= s[2]
        names = [("sw_power_cap", "nvmlClocksThrottleReasonSwPowerCap"),
                 ("hw_slowdown", "nvmlClocksThrottleReasonHwSlowdown"),
                 ("hw_thermal_slowdown", "nvmlClocksThrottleReasonHwThermalSlowdown"),
                 ("sw_thermal_slowdown", "nvmlClocksThrottleReasonSwThermalSlowdown"),
                 ("hw_power_brake", "nvmlClocksThrottleReasonHwPowerBrakeSlowdown")]
        reasons = [n for n, attr in names if bits & getattr(nv, attr, 0)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(inside), "power_w_max": round(max(s[3] for s in inside), 1)}


# ---- building the workload --------------------------------------------------------------------------
def build_handle(name, units=None):
    """Task -> KernelHandle for a configuration, through the reference-facing interface, with the
    library's default knobs (an empty knob dict)."""
    from heron_b200.config import Config
    from heron_b200.ops import cuda as heron_cuda, x86 as heron_cpu
    from heron_b200.task import KernelHandle, Task
    from heron_b200.workloads import CONFIGS
    cfg = CONFIGS[name]
    case = list(cfg["case"])
    if units is not None:
        case[0] = units
    registry, codegen = (heron_cpu, "CPU") if cfg["platform"] == "dlboost" else (heron_cuda, "GPU_TENSOR_CORE")
    t = Task(name, registry.getOpFromName(cfg["op"]), case + [cfg["in_dtype"], cfg["out_dtype"]], "cuda")
    c = Config()
    c.codegen_type, c.log_dir = codegen, None
    t.config = c
    outs = t.getOut()
    args = outs[0].op.input_tensors + outs
    if "w_dtype" in cfg:
        args[1].dtype = cfg["w_dtype"]
    return KernelHandle(outs[0].op, {}), args


def to_dev(a, device):
    import numpy as np
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from heron_b200 import _lib
    from heron_b200.kernels import TORCH_DTYPES
    from heron_b200.multi import partition
    from heron_b200.runner.host_pipeline import HostPipeline
    from heron_b200.workloads import CONFIGS, make_inputs, work_and_bytes

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torch.distributed.run with %d ranks" % (args.gpus, args.gpus))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # keep stdout to the one JSON line: NCCL's version banner goes to stdout at VERSION level
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=device)

    name = args.workload
    cfg = CONFIGS[name]
    shards = cfg["op"] != "gemm" and world > 1
    units_total = cfg["case"][0]
    if shards:
        start, count = partition(units_total, world)[rank]
        units = count
        host_in = make_inputs(name, shard=(start, count))
        scaling = "strong"
    else:
        units = None
        host_in = make_inputs(name)
        scaling = "weak"
    handle, targs = build_handle(name, units)
    work, alg_bytes = work_and_bytes(name, units)
    total_work = work_and_bytes(name)[0] * (1 if shards or world == 1 else world)

    # Rotating buffer sets: more bytes than L2 (126 MB) between two uses of the same set.
    set_bytes = sum(int(np.prod(a.shape)) * torch.empty(0, dtype=TORCH_DTYPES[a.dtype]).element_size() for a in targs)
    n_sets = max(2, min(16, int(np.ceil(300e6 / max(set_bytes, 1))) + 1))
    sets = []
    for _ in range(n_sets):
        ins = [to_dev(h, device) for h in host_in]
        out = torch.empty(targs[-1].shape, dtype=TORCH_DTYPES[targs[-1].dtype], device=device)
        sets.append(handle.plan(*ins, out))
    l2_note = "rotating %d buffer sets of %.0f MB (> 126 MB L2 between reuses)" % (n_sets, set_bytes / 1e6)
    if n_sets * set_bytes < 260e6:
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    else:
        flush = None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(args.warmup):
        sets[i % n_sets].launch()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        if flush is not None:
            flush.zero_()
        sets[i % n_sets].launch()
    e1.record()
    barrier()
    t1 = time.perf_counter()
    elapsed_ms = e0.elapsed_time(e1)
    if flush is not None:
        # cost of the flush writes alone, measured the same way and subtracted
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for i in range(args.steps):
            flush.zero_()
        f1.record()
        torch.cuda.synchronize(device)
        elapsed_ms = max(elapsed_ms - f0.elapsed_time(f1), 1e-6)
        l2_note = "L2 flushed by a 256 MB write before every step (its cost measured and subtracted)"
    clocks = sampler.summary(t0, t1)
    status = _lib.last_status()
    if status != 0:
        raise SystemExit("kernel status %d (%s)" % (status, _lib.status_string(status)))

    # ---- end to end through host buffers ---------------------------------------------------------
    resident = (1,) if cfg["op"].startswith("c2d") else ()
    pipe = HostPipeline(handle, targs, depth=2, device_id=local_rank, resident=resident)
    pinned = [torch.from_numpy(np.ascontiguousarray(h)).pin_memory() for h in host_in]
    pipe.upload_resident(pinned)
    e2e_steps = max(3, min(args.steps, 20 if set_bytes > 50e6 else 200))
    for _ in range(2):
        pipe.wait(pipe.submit(pinned))
    barrier()
    w0 = time.perf_counter()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    slots = []
    checksum = 0.0
    for i in range(e2e_steps):
        if len(slots) >= pipe.depth:
            res = pipe.wait(slots.pop(0))
            checksum += float(res.view(-1)[0])
        slots.append(pipe.submit(pinned))
    for s in slots:
        checksum += float(pipe.wait(s).view(-1)[0])
    pipe.drain()
    g1.record()
    torch.cuda.synchronize(device)
    e2e_ms = max(g0.elapsed_time(g1), (time.perf_counter() - w0) * 1e3) / e2e_steps
    barrier()

    # ---- sharded runs: compute + in-place all-gather of the whole output, reported separately ------
    gather_ms = 0.0
    if shards:
        from heron_b200.multi import gather_output, shard_slice
        full_shape = (units_total,) + tuple(targs[-1].shape[1:])
        full = torch.empty(full_shape, dtype=TORCH_DTYPES[targs[-1].dtype], device=device)
        gplan = handle.plan(*[to_dev(h, device) for h in host_in], shard_slice(full, rank, world))
        gsteps = max(3, min(args.steps, 50))
        for _ in range(3):
            gplan.launch()
            gather_output(full, rank, world)
        barrier()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record()
        for _ in range(gsteps):
            gplan.launch()
            gather_output(full, rank, world)
        h1.record()
        barrier()
        gather_ms = h0.elapsed_time(h1) / gsteps
        gather_bytes = full.numel() * full.element_size()

    times = torch.tensor([elapsed_ms, e2e_ms, gather_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, gather_ms = float(times[0]), float(times[1]), float(times[2])
    ms_per_step = elapsed_ms / args.steps

    if rank == 0:
        peaks = load_peaks()
        unit = "TFLOP/s" if cfg["in_dtype"] == "float16" else "TOP/s"
        value = total_work / (ms_per_step * 1e-3) / 1e12
        per_launch_s = ms_per_step * 1e-3
        bound = "hbm" if name == "cfg4_bmm_s8_attention" else "tensor"
        sustained = elapsed_ms > 500.0
        if bound == "tensor":
            peak_key = "bf16_tflops_sustained" if sustained else "bf16_tflops"
            peak = peaks[peak_key] * (2.0 if cfg["in_dtype"] != "float16" else 1.0)
            achieved = work / per_launch_s / 1e12
            peak_note = "%s %s cuBLAS bf16 %s%s" % (
                peaks["_source"], "sustained" if sustained else "burst", peak_key,
                " x2 (int8 runs at twice the bf16 rate; no int8 peak was measured)" if cfg["in_dtype"] != "float16" else "")
            runit = unit
        else:
            peak = peaks["hbm_gbs"]
            achieved = alg_bytes / per_launch_s / 1e9
            peak_note = "%s STREAM-style copy hbm_gbs" % peaks["_source"]
            runit = "GB/s"
        line = {
            "metric": METRIC, "value": round(value, 3), "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 6), "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": arithmetic_dtype(cfg), "data": "synthetic",
            "config": {"workload": name, "op": cfg["op"], "case": cfg["case"], "l2": l2_note,
                       "knobs": sets[0].knobs(),
                       "multi_gpu": ("replicas only: this operator has no batch-like dimension" if not shards and world > 1
                                     else ("leading dimension split over ranks, no collective" if shards else "single GPU"))},
            "roofline": {"bound": bound, "achieved": round(achieved, 2), "peak": round(peak, 1), "unit": runit,
                         "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC_BYTES.get(name),
                         "peak_source": peak_note,
                         "algorithmic_per_launch": {"ops": work, "bytes": alg_bytes}},
            "clocks": clocks,
            "e2e": {"value": round(total_work / (e2e_ms * 1e-3) / 1e12, 4), "unit": unit,
                    "h2d_bytes_per_step": pipe.h2d_bytes_per_step, "d2h_bytes_per_step": pipe.d2h_bytes_per_step,
                    "ms_per_step": round(e2e_ms, 4), "steps": e2e_steps,
                    "how": "pinned host inputs -> device -> kernel -> pinned host output every step, "
                           "3-stream pipeline of depth 2"},
            "gpu_launches": args.steps,  # one kernel per step
        }
        if shards:
            line["config"]["with_all_gather"] = {
                "ms_per_step": round(gather_ms, 5),
                "note": "kernel writes its shard into the full buffer, then one in-place NCCL all-gather; "
                        "%.1f MB gathered per step" % (gather_bytes / 1e6)}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(name, budget_s=args.cpu_seconds)
        emit(line)
    sampler.stop()
    if world > 1:
        dist.destroy_process_group()


# ---- CPU legs ----------------------------------------------------------------------------------------
def cpu_problem(name, steps=10):
    """(callable running one bounded sample on the host cores, ops of that sample, description).
    The sample shrinks as ``steps`` grows so that a whole run stays within a few minutes."""
    import numpy as np
    from heron_b200.workloads import CONFIGS, make_inputs
    from oracle import dlboost as dl, np_oracle as npo
    cfg = CONFIGS[name]
    case = cfg["case"]
    if name == "cfg2_gemm_f16_4096":
        a, b = make_inputs(name)
        rows = 512 if steps <= 100 else (64 if steps <= 1000 else 16)
        g = dl.GemmF16(rows, 4096, 4096)
        a = np.ascontiguousarray(a[:rows])
        return (lambda: g(a, b)), 2 * rows * 4096 * 4096, \
            "fp32 AVX512 port (the reference has no fp16 x86 operator): rows 0..%d of A against all of B" % (rows - 1)
    if name == "cfg1_gemm_u8s8_64":
        a, b = make_inputs(name)
        g = dl.GemmU8S8(64, 64, 64)
        return (lambda: g(a, b)), 2 * 64 ** 3, "the whole 64^3 problem per call"
    if name == "cfg4_bmm_s8_attention":
        nb = 24 if steps <= 100 else 2
        a, b = make_inputs(name, shard=(0, nb))
        g = dl.BmmS8S8(nb, 512, 64, 512)
        return (lambda: g(a, b)), 2 * nb * 512 * 512 * 64, \
            "batches 0..%d of 192; s8 x s8 through the u8 x s8 VNNI kernel with the +128 bias correction" % (nb - 1)
    if name == "cfg5_conv_u8s8_resnet_s4":
        ni = 32 if steps <= 100 else 2
        x, w = make_inputs(name, shard=(0, ni))
        wp = npo.pack_filter_x86(w, 64)
        g = dl.ConvPacked(ni, 7, 7, 512, 512, 3, 3, 1, 1, 1, 64)
        return (lambda: g(x, wp)), 2 * ni * 49 * 512 * 4608, "images 0..%d of 1024, OhwI64o4i filter" % (ni - 1)
    if name == "cfg3_conv_f16_resnet_s2":
        # im2col + the fp32 GEMM port on one image's worth of rows at a time
        x, w = make_inputs(name, shard=(0, 2))
        cols, _ = npo._im2col(x, 3, 3, 1, 1, 1)
        wt = np.ascontiguousarray(w.reshape(576, 64).T)
        g = dl.GemmF16(cols.shape[0], 576, 64)
        return (lambda: g(cols, wt)), 2 * cols.shape[0] * 576 * 64, \
            "images 0..1 of 32 as an explicit-im2col fp32 GEMM (the reference has no fp16 x86 operator)"
    raise KeyError(name)


def time_cpu(fn, budget_s, min_calls=3):
    fn()
    t0 = time.perf_counter()
    calls = 0
    while calls < min_calls or (time.perf_counter() - t0) < budget_s:
        fn()
        calls += 1
        if calls >= 100000:
            break
    return (time.perf_counter() - t0) / calls, calls


def cpu_baseline(name, budget_s=8.0):
    from heron_b200.workloads import CONFIGS
    from oracle import dlboost as dl
    dl.set_threads(os.cpu_count() or 1)
    fn, ops, sample = cpu_problem(name)
    sec, calls = time_cpu(fn, budget_s)
    unit = "TFLOP/s" if CONFIGS[name]["in_dtype"] == "float16" else "TOP/s"
    return {"value": round(ops / sec / 1e12, 5), "unit": unit, "cores": dl.max_threads(), "kind": "port",
            "sample": "%s; %d calls, %.3f ms each; host has %d logical CPUs; AVX512-VNNI %s"
                      % (sample, calls, sec * 1e3, os.cpu_count(), "yes" if dl.has_vnni() else "no (scalar twin)")}


def run_reference(args):
    """The reference arm: the CPU port of the reference's x86 program structure on this box's host
    cores (the reference itself needs Apache TVM, which is not installed and cannot be)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from heron_b200.workloads import CONFIGS
    from oracle import dlboost as dl
    dl.set_threads(os.cpu_count() or 1)  # torch.distributed.run exports OMP_NUM_THREADS=1
    name = args.workload
    cfg = CONFIGS[name]
    fn, ops, sample = cpu_problem(name, args.steps)
    for _ in range(max(args.warmup, 1)):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    sec = (time.perf_counter() - t0) / args.steps
    unit = "TFLOP/s" if cfg["in_dtype"] == "float16" else "TOP/s"
    value = round(ops / sec / 1e12, 5)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": unit,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(sec * 1e3, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": arithmetic_dtype(cfg), "data": "synthetic",
        "config": {"workload": name, "op": cfg["op"], "case": cfg["case"],
                   "note": "each step is a bounded sample of the workload: " + sample},
        "cpu_baseline": {"value": value, "unit": unit, "cores": dl.max_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Whatever libraries print (NCCL's version banner is a C-level write to stdout) goes to stderr;
    the descriptor stdout had is kept for the one JSON line."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=8.0)
    args = ap.parse_args()
    keep_stdout_for_the_result()
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 10
        args.warmup = args.warmup if args.warmup is not None else 3
        run_reference(args)
    else:
        args.steps = args.steps if args.steps is not None else 5000
        args.warmup = max(3, args.warmup if args.warmup is not None else 20)
        run_ours(args)


if __name__ == "__main__":
    main()
