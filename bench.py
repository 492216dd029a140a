#!/usr/bin/env python
"""Benchmark of the hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step is one pass of one operator over one batch of seeded synthetic input.  The default
workload is the int8 NHWC conv of ResNet-50 stage 4 at N = 1024 images: the largest of the five
benchmark configurations (heron_b200/workloads.py) that fits one GPU, tensor-bound, and one of
the two whose leading dimension shards.

With N > 1 (launched under torch.distributed.run, one rank per GPU) the images (conv) or batches
(batched GEMM) are split over the ranks with no data-path collective: total work is fixed
("strong" scaling), `value` = total work / slowest rank's device time.  Before timing, the ranks
gather their shards once and rank 0 checks the whole output with exact integer sum identities
(`sharded_check`).  A GEMM workload has nothing to shard and runs as independent replicas.

Rank 0 prints ONE JSON line.  At N = 1 it carries a `per_config` block with the other four
configurations (device-timed value, roofline, end-to-end and CPU baseline each); at N > 1 a
`sharded` block with compute-only and compute + all-gather times of both sharded configurations.

`--impl reference` times the CPU port of the reference's x86 program structure
(oracle/dlboost_baseline.c) on the host cores instead; together with the `cpu_baseline` legs it
is the only code in this file that executes anything under oracle/ (besides `sharded_check`,
which uses no oracle code at all: its identities are evaluated with numpy).
"""
import argparse
import json
import os
import sys
import threading
import time

# (before torch is imported: the symmetric-memory allocations of the sharded block bind nothing to
# an NVLink multicast object; a rank that dies while bound to one disturbs the box's other GPUs)
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "per-op TFLOPS/TOPS & % of B200 dense peak at 1/2/4/8 GPUs"
DEFAULT_WORKLOAD = "cfg5_conv_u8s8_resnet_s4"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# Nominal dense figures of one B200 (HGX): fp16 / int8 tensor throughput and HBM3e bandwidth.
NOMINAL = {"f16_tflops": 2250.0, "i8_tops": 4500.0, "hbm_gbs": 7700.0}
# Which bound each configuration's dominant kernel is held against (both for the ridge case).
BOUNDS = {
    "cfg1_gemm_u8s8_64": ("hbm",),
    "cfg2_gemm_f16_4096": ("tensor",),
    "cfg3_conv_f16_resnet_s2": ("hbm", "tensor"),
    "cfg4_bmm_s8_attention": ("hbm",),
    "cfg5_conv_u8s8_resnet_s4": ("tensor",),
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


def load_traffic():
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of each configuration's
    dominant kernel, from the table kept beside the ncu summaries it was read from."""
    table = {}
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    if os.path.exists(path):
        for row in open(path):
            f = row.split()
            if len(f) >= 3 and not row.startswith("#"):
                table[f[0]] = {"bytes": float(f[1]), "commit": f[2], "source": " ".join(f[3:])}
    return table


def arithmetic_dtype(cfg):
    return {"float16": "f16 (fp32 accumulate)", "int8": "s8 (s32 accumulate)",
            "uint8": "u8 x s8 (s32 accumulate)"}[cfg["in_dtype"]]


# ---- clocks -------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons of one GPU through NVML (read-only calls) while
    a timed region runs.  The NVML handle is looked up by the CUDA device's UUID: NVML indices
    ignore CUDA_VISIBLE_DEVICES, so an index could name another tenant's GPU."""

    def __init__(self, cuda_index, period=0.01):
        super().__init__(daemon=True)
        self.period = period
        self.samples = []
        self._stop_flag = threading.Event()
        self.why = None
        self.nv = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except TypeError:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.nv = pynvml
        except Exception as e:  # no pynvml, no NVML library, or the device is not visible to NVML
            self.why = "nvml unavailable: %s: %s" % (type(e).__name__, e)

    def sample(self):
        """One synchronous sample (also used right before and after a timed region)."""
        if self.nv is None:
            return
        nv = self.nv
        try:
            mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
            reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
            self.samples.append((time.perf_counter(), mhz, reasons, watts))
        except Exception as e:
            self.why = "nvml sample failed: %s" % e

    def run(self):
        while self.nv is not None and not self._stop_flag.is_set():
            self.sample()
            time.sleep(self.period)

    def stop(self):
        self._stop_flag.set()

    def summary(self, t0, t1, device_ms=None):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.why or "nvml unavailable"]}
        nv = self.nv
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        note = None
        if not inside:
            # a region shorter than the sampling period: the samples taken right before and after it
            near = sorted(self.samples, key=lambda s: min(abs(s[0] - t0), abs(s[0] - t1)))[:2]
            if not near:
                return {"sm_mhz": None, "sm_max_mhz": self.max_mhz,
                        "reasons": [self.why or "no sample in timed region"]}
            inside, note = near, "no sample in timed region: the nearest samples around it"
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
        out = {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
               "samples": len(inside), "power_w_max": round(max(s[3] for s in inside), 1)}
        if device_ms is not None:
            out["ms_per_step_x_sm_mhz"] = round(device_ms * out["sm_mhz"], 3)
        if note:
            out["note"] = note
        return out


# ---- building a workload ---------------------------------------------------------------------------
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


class Env:
    """Process-wide state of a bench run: ranks, device, barrier."""

    def __init__(self, gpus):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != gpus and self.world == 1 and gpus > 1:
            raise SystemExit("--gpus %d needs torch.distributed.run with %d ranks" % (gpus, gpus))
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            # keep stdout to the one JSON line: NCCL's version banner goes to stdout at VERSION level
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.device)

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, dtype=self.torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]


def time_device(env, name, steps, warmup, sampler=None):
    """Device-timed steps of one configuration (this rank's shard of it when it shards and there
    is more than one rank).  Returns a dict with ms_per_step (this rank), knobs, notes."""
    import numpy as np
    torch = env.torch
    from heron_b200 import _lib
    from heron_b200.kernels import TORCH_DTYPES
    from heron_b200.multi import partition
    from heron_b200.workloads import CONFIGS, make_inputs, work_and_bytes
    cfg = CONFIGS[name]
    shards = cfg["op"] != "gemm" and env.world > 1
    units = None
    if shards:
        start, units = partition(cfg["case"][0], env.world)[env.rank]
        host_in = make_inputs(name, shard=(start, units))
    else:
        host_in = make_inputs(name)
    handle, targs = build_handle(name, units)
    work, alg_bytes = work_and_bytes(name, units)

    # Rotating buffer sets: more bytes than L2 (126 MB) between two uses of the same set.
    set_bytes = sum(int(np.prod(a.shape)) * torch.empty(0, dtype=TORCH_DTYPES[a.dtype]).element_size() for a in targs)
    n_sets = max(2, min(16, int(np.ceil(300e6 / max(set_bytes, 1))) + 1))
    sets = []
    for _ in range(n_sets):
        ins = [to_dev(h, env.device) for h in host_in]
        out = torch.empty(targs[-1].shape, dtype=TORCH_DTYPES[targs[-1].dtype], device=env.device)
        sets.append(handle.plan(*ins, out))
    l2_note = "rotating %d buffer sets of %.1f MB (> 126 MB L2 between reuses)" % (n_sets, set_bytes / 1e6)
    flush = None
    if n_sets * set_bytes < 260e6:
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=env.device)

    for i in range(warmup):
        sets[i % n_sets].launch()
    env.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler is not None:
        sampler.sample()
    t0 = time.perf_counter()
    pairs = []
    e0.record()
    for i in range(steps):
        if flush is not None:
            # a working set smaller than L2: flush before every step and put that step's launch
            # between events of its own (subtracting a separately timed flush loop from the whole
            # loop left a difference of two large numbers: 8 to 40 us for the same 6 us kernel)
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            sets[i % n_sets].launch()
            b.record()
            pairs.append((a, b))
        else:
            sets[i % n_sets].launch()
    e1.record()
    env.barrier()
    t1 = time.perf_counter()
    if sampler is not None:
        sampler.sample()
    elapsed_ms = e0.elapsed_time(e1)
    if flush is not None:
        elapsed_ms = max(sum(a.elapsed_time(b) for a, b in pairs), 1e-6)
        l2_note = "L2 flushed by a 256 MB write before every step; each step's launch timed between CUDA events of its own"
    status = _lib.last_status()
    if status != 0:
        raise SystemExit("kernel status %d (%s) in %s" % (status, _lib.status_string(status), name))
    return {"handle": handle, "targs": targs, "host_in": host_in, "units": units, "shards": shards,
            "work": work, "alg_bytes": alg_bytes, "elapsed_ms": elapsed_ms, "ms_per_step": elapsed_ms / steps,
            "l2": l2_note, "knobs": sets[0].knobs(), "set_bytes": set_bytes, "wall": (t0, t1)}


def time_e2e(env, name, dev_run, steps):
    """The same operator through host buffers: every step copies its inputs from pinned host memory
    to the device, launches, and copies the output back to pinned host memory."""
    import numpy as np
    torch = env.torch
    from heron_b200.runner.host_pipeline import HostPipeline
    from heron_b200.workloads import CONFIGS
    cfg = CONFIGS[name]
    resident = (1,) if cfg["op"].startswith("c2d") else ()
    pipe = HostPipeline(dev_run["handle"], dev_run["targs"], depth=2, device_id=env.local_rank, resident=resident)
    pinned = [torch.from_numpy(np.ascontiguousarray(h)).pin_memory() for h in dev_run["host_in"]]
    pipe.upload_resident(pinned)
    e2e_steps = max(3, min(steps, 20 if dev_run["set_bytes"] > 50e6 else 200))
    for _ in range(2):
        pipe.wait(pipe.submit(pinned))
    env.barrier()
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
    torch.cuda.synchronize(env.device)
    e2e_ms = max(g0.elapsed_time(g1), (time.perf_counter() - w0) * 1e3) / e2e_steps
    env.barrier()
    return {"ms_per_step": e2e_ms, "steps": e2e_steps, "h2d": pipe.h2d_bytes_per_step, "d2h": pipe.d2h_bytes_per_step}


def roofline_of(name, work, alg_bytes, per_launch_s, sustained, peaks, traffic):
    """roofline objects of one configuration's kernel: the first is the binding one."""
    from heron_b200.workloads import CONFIGS
    cfg = CONFIGS[name]
    int8 = cfg["in_dtype"] != "float16"
    out = []
    for bound in BOUNDS[name]:
        if bound == "tensor":
            peak_key = "bf16_tflops_sustained" if sustained else "bf16_tflops"
            peak = peaks[peak_key] * (2.0 if int8 else 1.0)
            nominal = NOMINAL["i8_tops"] if int8 else NOMINAL["f16_tflops"]
            achieved = work / per_launch_s / 1e12
            unit = "TOP/s" if int8 else "TFLOP/s"
            note = "%s %s cuBLAS bf16 (%s)%s" % (
                peaks["_source"], "sustained" if sustained else "burst", peak_key,
                " x2: int8 MMA runs at twice the bf16 rate and no int8 peak was measured" if int8 else "")
        else:
            peak, nominal = peaks["hbm_gbs"], NOMINAL["hbm_gbs"]
            achieved = alg_bytes / per_launch_s / 1e9
            unit = "GB/s"
            note = "%s STREAM-style copy (hbm_gbs)" % peaks["_source"]
        t = traffic.get(name)
        r = {"bound": bound, "achieved": round(achieved, 2), "peak": round(peak, 1), "unit": unit,
             "frac": round(achieved / peak, 4), "of": "of %s" % peaks["_source"],
             "frac_nominal": round(achieved / nominal, 4), "nominal_peak": nominal,
             "traffic": t["bytes"] if t else None,
             "traffic_source": ("%s @ %s" % (t["source"], t["commit"])) if t else None,
             "peak_source": note, "launch_us": round(per_launch_s * 1e6, 3),
             "algorithmic_per_launch": {"ops": work, "bytes": alg_bytes}}
        if name == "cfg1_gemm_u8s8_64":
            r["note"] = "one 64^3 tile: bound by launch latency, the fraction says nothing about the kernel"
        out.append(r)
    return out


def is_sustained(elapsed_ms, clocks):
    """Which measured peak a timed region is held against: the sustained one when the region was
    long (over half a second) or ran under the power cap (`sw_power_cap` active in its clock
    record: on this part the cap bites after some 50 ms of tensor work and costs 10-15 %), else the
    burst one.  The two cuBLAS figures in MEASURED_PEAKS.json were taken in exactly these regimes."""
    return elapsed_ms > 500.0 or "sw_power_cap" in clocks.get("reasons", [])


def unit_of(cfg):
    return "TFLOP/s" if cfg["in_dtype"] == "float16" else "TOP/s"


# ---- sharded runs -----------------------------------------------------------------------------------
def sum_identity_check(name, full_host):
    """Exact integer identities over every element of a whole int32 output, evaluated with numpy from
    the seeded inputs: conv: sum_f out[n,y,x,f] = conv(in, sum_f w); bmm: row and column sums."""
    import numpy as np
    from heron_b200.workloads import CONFIGS, make_inputs
    cfg = CONFIGS[name]
    got = full_host.astype(np.int64)
    if cfg["op"] == "bmm":
        a, b = make_inputs(name)
        a64, b64 = a.astype(np.int64), b.astype(np.int64)
        return bool(np.array_equal(got.sum(axis=2), np.einsum("bik,bk->bi", a64, b64.sum(axis=1))) and
                    np.array_equal(got.sum(axis=1), np.einsum("bjk,bk->bj", b64, a64.sum(axis=1))))
    x, w = make_inputs(name)
    N, H, W, CI, CO, KH, KW, s, p, d = cfg["case"]
    wsum = w.astype(np.int64).sum(axis=3)
    xp = np.pad(x.astype(np.int64), ((0, 0), (p, p), (p, p), (0, 0)))
    HO, WO = got.shape[1], got.shape[2]
    want = np.zeros(got.shape[:3], dtype=np.int64)
    for ry in range(KH):
        for rx in range(KW):
            win = xp[:, ry * d:ry * d + (HO - 1) * s + 1:s, rx * d:rx * d + (WO - 1) * s + 1:s, :]
            want += (win * wsum[ry, rx]).sum(axis=3)
    return bool(np.array_equal(got.sum(axis=3), want))


def run_sharded(env, name, steps):
    """compute-only and compute + all-gather of the whole output for one sharded configuration,
    after one checked gather.  Every rank's kernel writes into its slice(s) of a full-size buffer;
    the gather is in place.  With `chunks` > 1 the leading dimension is first cut into that many
    super-chunks, each split over the ranks, so that the gather of one super-chunk (second stream)
    overlaps the compute of the next."""
    torch, dist = env.torch, env.dist
    from heron_b200.kernels import TORCH_DTYPES
    from heron_b200.multi import ChunkedGather
    from heron_b200.workloads import CONFIGS, make_inputs, work_and_bytes
    cfg = CONFIGS[name]
    total = cfg["case"][0]
    out = {}
    for chunks in (1, 2, 4):
        cg = ChunkedGather(total, env.rank, env.world, chunks)
        probe_handle, probe_args = build_handle(name, cg.parts[0][1])
        full = torch.empty((total,) + tuple(probe_args[-1].shape[1:]),
                           dtype=TORCH_DTYPES[probe_args[-1].dtype], device=env.device)
        full.view(torch.uint8).fill_(0xCD)
        plans = []
        for (start, count) in cg.parts:
            handle, _ = build_handle(name, count)
            ins = [to_dev(h, env.device) for h in make_inputs(name, shard=(start, count))]
            plans.append(handle.plan(*ins, full[start:start + count]))
        cg.run(plans, full)
        env.barrier()
        if chunks == 1:
            ok = True
            if env.rank == 0:
                ok = sum_identity_check(name, full.cpu().numpy())
            flag = torch.tensor([1 if ok else 0], device=env.device)
            dist.broadcast(flag, src=0)
            out["sharded_check"] = "pass" if int(flag[0]) == 1 else "fail"
        gsteps = max(3, min(steps, 50))
        for _ in range(3):
            cg.run(plans, full)
        env.barrier()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record()
        for _ in range(gsteps):
            cg.run(plans, full)
        h1.record()
        env.barrier()
        ms = env.max_over_ranks([h0.elapsed_time(h1) / gsteps])[0]
        out["with_all_gather_ms_chunks%d" % chunks] = round(ms, 5)
        if chunks == 1:
            # compute alone on the same plan (the shard written into the full buffer)
            for _ in range(3):
                plans[0].launch()
            env.barrier()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record()
            for _ in range(gsteps * 4):
                plans[0].launch()
            c1.record()
            env.barrier()
            cms = env.max_over_ranks([c0.elapsed_time(c1) / (gsteps * 4)])[0]
            out["compute_ms"] = round(cms, 5)
            out["compute_value"] = round(work_and_bytes(name)[0] / (cms * 1e-3) / 1e12, 3)
            out["gathered_mb"] = round(full.numel() * full.element_size() / 1e6, 1)
        del plans, full
    # No collective: every rank's kernel stores its shard into every rank's copy of the output
    # (symmetric memory; TMA stores from the kernel's staging buffer over NVLink), then a
    # one-element all-reduce on the stream as the barrier.
    try:
        from heron_b200.multi import PeerStoreOutput, partition
        start, count = partition(total, env.world)[env.rank]
        handle, hargs = build_handle(name, count)
        po = PeerStoreOutput((total,) + tuple(hargs[-1].shape[1:]), TORCH_DTYPES[hargs[-1].dtype], env.device)
        po.full.view(torch.uint8).fill_(0xCD)
        po.barrier()
        ins = [to_dev(h, env.device) for h in make_inputs(name, shard=(start, count))]
        plan = po.attach(handle.plan(*ins, po.mine(start, count)), start, count)
        plan.launch()
        po.barrier()
        env.barrier()
        ok = True
        if env.rank == env.world - 1:  # (a rank other than the one that checked the gathered form)
            ok = sum_identity_check(name, po.full.cpu().numpy())
        flag = torch.tensor([1 if ok else 0], device=env.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        out["peer_store_check"] = "pass" if int(flag[0]) == 1 else "fail"
        out["peer_store_multicast_bound"] = bool(getattr(po._hdl, "multicast_ptr", 0))
        gsteps = max(3, min(steps, 50))
        for _ in range(3):
            plan.launch()
            po.barrier()
        env.barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(gsteps):
            plan.launch()
            po.barrier()
        p1.record()
        env.barrier()
        out["with_peer_stores_ms"] = round(env.max_over_ranks([p0.elapsed_time(p1) / gsteps])[0], 5)
        del plan, po
    except Exception as e:  # symmetric memory unavailable on this box: the gathered form stands
        out["with_peer_stores_ms"] = None
        out["peer_store_note"] = "%s: %s" % (type(e).__name__, str(e)[:160])
    best = min(v for k, v in out.items() if k.startswith("with_all_gather_ms"))
    out["with_all_gather_ms"] = best
    out["unit"] = unit_of(cfg)
    out["note"] = ("compute_ms: this configuration's shard kernel alone (L2-warm, same buffers every launch); "
                   "with_all_gather_ms: kernels write their shards into the full buffer, in-place NCCL all-gather, "
                   "best of 1 / 2 / 4 overlapped super-chunks; with_peer_stores_ms: no collective, every rank's kernel "
                   "stores its tiles into every rank's buffer (hb_plan_set_peer_outputs) + a one-element all-reduce as the barrier")
    return out


def run_ours(args):
    import torch  # noqa: F401
    from heron_b200.workloads import CONFIGS, work_and_bytes

    env = Env(args.gpus)
    name = args.workload
    cfg = CONFIGS[name]
    peaks, traffic = load_peaks(), load_traffic()

    sharded_block = None
    if env.world > 1 and cfg["op"] != "gemm":
        # correctness of the sharded path first, then its gather timings (both sharded configurations)
        sharded_block = {}
        for sname in ([name] + [n for n in ("cfg5_conv_u8s8_resnet_s4", "cfg4_bmm_s8_attention") if n != name]):
            sharded_block[sname] = run_sharded(env, sname, args.steps)

    sampler = ClockSampler(env.local_rank)
    sampler.start()
    dev_run = time_device(env, name, args.steps, args.warmup, sampler)
    elapsed_ms = env.max_over_ranks([dev_run["elapsed_ms"]])[0]
    ms_per_step = elapsed_ms / args.steps
    clocks = sampler.summary(dev_run["wall"][0], dev_run["wall"][1], ms_per_step)
    sampler.stop()
    e2e = time_e2e(env, name, dev_run, args.steps)
    e2e_ms = env.max_over_ranks([e2e["ms_per_step"]])[0]

    shards = dev_run["shards"]
    total_work = work_and_bytes(name)[0] * (1 if shards or env.world == 1 else env.world)
    scaling = "strong" if (shards or cfg["op"] != "gemm") else "weak"

    per_config = None
    if env.world == 1 and not args.only_default:
        per_config = {}
        for other in CONFIGS:
            if other == name:
                continue
            ocfg = CONFIGS[other]
            osteps = min(args.steps, 2000)
            osampler = ClockSampler(env.local_rank, period=0.005)
            osampler.start()
            r = time_device(env, other, osteps, max(3, min(args.warmup, 20)), osampler)
            oclocks = osampler.summary(r["wall"][0], r["wall"][1], r["ms_per_step"])
            osampler.stop()
            oe = time_e2e(env, other, r, osteps)
            rl = roofline_of(other, r["work"], r["alg_bytes"], r["ms_per_step"] * 1e-3,
                             is_sustained(r["elapsed_ms"], oclocks), peaks, traffic)
            entry = {
                "value": round(r["work"] / (r["ms_per_step"] * 1e-3) / 1e12, 4), "unit": unit_of(ocfg),
                "ms_per_step": round(r["ms_per_step"], 6), "steps": osteps, "dtype": arithmetic_dtype(ocfg),
                "config": {"workload": other, "op": ocfg["op"], "case": ocfg["case"]},
                "roofline": rl[0],
                "clocks": oclocks,
                "e2e": {"value": round(r["work"] / (oe["ms_per_step"] * 1e-3) / 1e12, 4), "unit": unit_of(ocfg),
                        "h2d_bytes_per_step": oe["h2d"], "d2h_bytes_per_step": oe["d2h"],
                        "ms_per_step": round(oe["ms_per_step"], 4), "steps": oe["steps"]},
                "details": {"l2": r["l2"], "knobs": r["knobs"]},
            }
            if len(rl) > 1:
                entry["roofline_" + rl[1]["bound"]] = rl[1]
            if not args.no_cpu_baseline:
                entry["cpu_baseline"] = cpu_baseline(other, budget_s=min(args.cpu_seconds, 3.0))
            per_config[other] = entry
            del r

    if env.rank == 0:
        unit = unit_of(cfg)
        value = total_work / (ms_per_step * 1e-3) / 1e12
        rl = roofline_of(name, dev_run["work"], dev_run["alg_bytes"], ms_per_step * 1e-3,
                         is_sustained(elapsed_ms, clocks), peaks, traffic)
        line = {
            "metric": METRIC, "value": round(value, 3), "unit": unit, "n_gpus": env.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 6), "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": arithmetic_dtype(cfg), "data": "synthetic",
            "config": {"workload": name, "op": cfg["op"], "case": cfg["case"]},
            "details": {
                "l2": dev_run["l2"], "knobs": dev_run["knobs"],
                "multi_gpu": ("single GPU" if env.world == 1 else
                              ("leading dimension split over %d ranks (%s units each), no data-path collective; "
                               "roofline is one rank's kernel on its shard" % (env.world, dev_run["units"]) if shards
                               else "replicas only: this operator has no batch-like dimension")),
            },
            "roofline": rl[0],
            "clocks": clocks,
            "e2e": {"value": round(total_work / (e2e_ms * 1e-3) / 1e12, 4), "unit": unit,
                    "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                    "ms_per_step": round(e2e_ms, 4), "steps": e2e["steps"],
                    "how": "pinned host inputs -> device -> kernel -> pinned host output every step (per rank: "
                           "its shard), 3-stream pipeline of depth 2"},
            "gpu_launches": args.steps,  # one kernel of this library per step
        }
        if len(rl) > 1:
            line["roofline_" + rl[1]["bound"]] = rl[1]
        if sharded_block is not None:
            line["sharded_check"] = ("pass" if all(v.get("sharded_check") == "pass" for v in sharded_block.values())
                                     else "fail")
            line["sharded"] = sharded_block
        if env.world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(name, budget_s=args.cpu_seconds)
        if per_config is not None:
            line["per_config"] = per_config
        emit(line)
    if env.world > 1:
        env.dist.destroy_process_group()


# ---- CPU legs ----------------------------------------------------------------------------------------
def cpu_problem(name, steps=10):
    """(callable running one bounded sample on the host cores, ops of that sample, description).
    The sample shrinks as ``steps`` grows so that a whole run stays within a few minutes."""
    import numpy as np
    from heron_b200.workloads import make_inputs
    from oracle import dlboost as dl, np_oracle as npo
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
    return {"value": round(ops / sec / 1e12, 5), "unit": unit_of(CONFIGS[name]), "cores": dl.max_threads(),
            "kind": "port",
            "sample": "%s; %d calls, %.3f ms each; host has %d logical CPUs; AVX512-VNNI %s"
                      % (sample, calls, sec * 1e3, os.cpu_count(), "yes" if dl.has_vnni() else "no (scalar twin)")}


def run_reference(args):
    """The reference arm: the CPU port of the reference's x86 program structure on this box's host
    cores (the reference itself needs Apache TVM, which is not installed and cannot be).  For the
    default workload that is a port of a reference program proper: the VNNI OhwI64o4i conv of
    ops/x86/conv2d_int8.py:31-93."""
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
    unit = unit_of(cfg)
    value = round(ops / sec / 1e12, 5)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": unit,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(sec * 1e3, 4), "higher_is_better": True,
        "scaling": "strong" if cfg["op"] != "gemm" else "weak", "vs_baseline": None,
        "dtype": arithmetic_dtype(cfg), "data": "synthetic",
        "config": {"workload": name, "op": cfg["op"], "case": cfg["case"]},
        "details": {"note": "each step is a bounded sample of the workload on the host cores: " + sample},
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
    ap.add_argument("--only-default", action="store_true",
                    help="skip the per_config block (the other four configurations) at N = 1")
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
