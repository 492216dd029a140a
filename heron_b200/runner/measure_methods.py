"""Timing of built kernels with CUDA events on the device
(the role of runner/measure_methods.py:106-188 in the reference, which times TVM modules with
``time_evaluator`` over RPC).

Protocol, mirroring the reference's: ``repeat`` groups of ``number`` back-to-back launches, each
group bracketed by two CUDA events on the launching stream; the cost of a group is its time
divided by ``number``; with more than two repeats the median is reported
(measure_methods.py:166-171).  ``min_repeat_ms`` grows ``number`` until a group lasts that long.
An optional L2 flush (a write over a buffer larger than L2) runs before every launch, with its
own cost measured and subtracted.  The error taxonomy keeps the reference's numbers: a wrong
result is error 100 (measure_methods.py:176-177), a device-side timeout or launch failure is a
run-time error, and a failed candidate scores perf 0 (runner/runner.py:13-18).
"""
import math
import time

import numpy as np


class MeasureErrorNo:
    NO_ERROR = 0
    INSTANTIATION_ERROR = 1
    COMPILE_HOST = 2
    COMPILE_DEVICE = 3
    RUNTIME_DEVICE = 4
    WRONG_ANSWER = 5
    BUILD_TIMEOUT = 6
    RUN_TIMEOUT = 7
    UNKNOWN_ERROR = 8
    HERON_WRONG_RESULT = 100


class MeasureResult:
    def __init__(self, costs, error_no, all_cost, timestamp):
        self.costs = costs
        self.error_no = error_no
        self.all_cost = all_cost
        self.timestamp = timestamp

    def __repr__(self):
        return "MeasureResult(costs=%s, error_no=%d)" % (self.costs, self.error_no)


L2_FLUSH_BYTES = 256 * 1024 * 1024

_flush_buf = {}


def _flush_buffer(device):
    import torch
    key = str(device)
    if key not in _flush_buf:
        _flush_buf[key] = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    return _flush_buf[key]


def time_launches(launch, number=3, repeat=4, min_repeat_ms=0, flush_l2=False, device=None, use_graph=True):
    """Seconds per launch for each of ``repeat`` groups.  ``launch()`` enqueues the kernel on the
    current stream.  Ten warm-up launches come first.

    A group of ``n`` launches is captured in a CUDA graph and replayed between the two events, so
    that the figure is the device's time per launch and not the host's enqueue rate (an operator
    here is one to three kernels of a few microseconds).  ``use_graph=False`` enqueues them one by
    one instead; that is also what happens if the capture fails."""
    import torch
    device = device or torch.device("cuda", torch.cuda.current_device())
    buf = _flush_buffer(device) if flush_l2 else None
    for _ in range(10):
        launch()
    torch.cuda.synchronize(device)
    graphs = {}

    def enqueue(n, with_kernel):
        for _ in range(n):
            if buf is not None:
                buf.zero_()
            if with_kernel:
                launch()

    def graph_for(n, with_kernel):
        key = (n, with_kernel)
        if key not in graphs:
            g = None
            if use_graph and n <= 4096:
                try:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        enqueue(n, with_kernel)
                    g.replay()
                    torch.cuda.synchronize(device)
                except Exception:
                    g = None
                    torch.cuda.synchronize(device)
            graphs[key] = g
        return graphs[key]

    def group(n, with_kernel):
        g = graph_for(n, with_kernel)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if g is not None:
            g.replay()
        else:
            enqueue(n, with_kernel)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) * 1e-3

    n = max(1, int(number))
    if min_repeat_ms > 0:
        while True:
            t = group(n, True)
            if t * 1e3 >= min_repeat_ms or n >= (1 << 20):
                break
            n = min(max(n + 1, int(n * min_repeat_ms / max(t * 1e3, 1e-3) * 1.1)), 1 << 20)
    costs = []
    for _ in range(int(repeat)):
        t = group(n, True)
        if buf is not None:
            t -= group(n, False)
        costs.append(max(t, 0.0) / n)
    return costs


def reduce_costs(costs):
    """The reference reports the median when it has more than two repeats."""
    costs = sorted(costs)
    return costs[len(costs) // 2] if len(costs) > 2 else float(np.mean(costs))


def perf_from_cost(seconds):
    """The reference's fitness encoding: ln(1 / seconds); 0 for a failed candidate."""
    return math.log(1.0 / seconds) if seconds and seconds > 0 else 0.0


def measure_handle(task, handle, args, number=3, repeat=4, min_repeat_ms=0, flush_l2=False, device_id=0):
    """Builds device buffers for ``args`` (random, or the task's reference inputs when a verify
    function is set), times the kernel, checks the result when asked to."""
    import torch
    from .. import _lib
    from ..kernels import TORCH_DTYPES
    tic = time.time()
    errno = MeasureErrorNo.NO_ERROR
    device = torch.device("cuda", device_id)
    try:
        with torch.cuda.device(device):
            if task.not_verify_correctness:
                tensors = []
                g = torch.Generator(device=device)
                g.manual_seed(0)
                for spec in args:
                    dt = TORCH_DTYPES[spec.dtype]
                    if dt.is_floating_point:
                        tensors.append(torch.randn(spec.shape, device=device, generator=g).to(dt))
                    else:
                        info = torch.iinfo(dt)
                        tensors.append(torch.randint(max(info.min, -128), min(info.max, 127) + 1, spec.shape,
                                                     device=device, generator=g, dtype=torch.int32).to(dt))
            else:
                tensors = [torch.from_numpy(np.ascontiguousarray(x)).to(device) for x in task.ref_input]
                out_spec = args[-1]
                tensors.append(torch.empty(out_spec.shape, dtype=TORCH_DTYPES[out_spec.dtype], device=device))
            plan = handle.plan(*tensors)
            costs = time_launches(plan.launch, number, repeat, min_repeat_ms, flush_l2, device)
            if _lib.last_status() != 0:
                raise _lib.HeronB200Error(_lib.HB_ERR_TIMEOUT, "kernel")
            cost = reduce_costs(costs)
            if not task.not_verify_correctness:
                got = tensors[-1].cpu().numpy()
                if not np.allclose(task.ref_output, got, rtol=task.rtol):
                    errno = MeasureErrorNo.HERON_WRONG_RESULT
            costs = (cost,)
    except _lib.HeronB200Error as exc:
        costs = (RuntimeError(str(exc)[:2048]),)
        errno = (MeasureErrorNo.INSTANTIATION_ERROR if exc.status in (_lib.HB_ERR_KNOB, _lib.HB_ERR_SHAPE)
                 else MeasureErrorNo.RUNTIME_DEVICE)
    tstamp = time.time()
    return MeasureResult(costs, errno, tstamp - tic, tstamp)
