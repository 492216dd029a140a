"""Runner: measures a batch of samples and records them (runner/runner.py:9-44 of the reference).

The reference hands ``MeasureInput``s to TVM's builder/runner pair; here each sample is
instantiated into a kernel handle and timed on the device with CUDA events
(measure_methods.measure_handle).  ``measure_option`` keeps the reference's knobs:
``number``, ``repeat``, ``min_repeat_ms``, ``timeout`` plus ``flush_l2`` and ``device_id``.
A ``measure_fn(task, handle, args) -> MeasureResult`` can be injected (tests use it to run the
whole tuning loop without a GPU).
"""
import math

import numpy as np

from .measure_methods import MeasureErrorNo, MeasureResult, measure_handle


class LocalRunner:
    """Counterpart of the reference's ``LocalRunner`` options object
    (tests/quick_start/dlboost/run.py:89-93)."""

    def __init__(self, number=3, repeat=4, min_repeat_ms=0, timeout=50, enable_cpu_cache_flush=False,
                 flush_l2=False, device_id=0):
        self.number, self.repeat, self.min_repeat_ms = number, repeat, min_repeat_ms
        self.timeout = timeout
        self.flush_l2 = flush_l2 or enable_cpu_cache_flush
        self.device_id = device_id


def measure_option(builder=None, runner=None):
    return {"builder": builder, "runner": runner or LocalRunner()}


class Runner:
    def __init__(self, measure_option, measure_fn=None):
        self.measure_option = measure_option
        self.measure_fn = measure_fn

    def results2tup(self, results):
        res = []
        for x in results:
            if x.error_no == 0:
                res.append((x.error_no, math.log(1 / float(np.array(x.costs).mean()))))
            else:
                res.append((x.error_no, 0.0))
        return res

    def measure_batch(self, samples):
        opt = self.measure_option["runner"]
        out = []
        for sample in samples:
            task = sample.task
            try:
                handle, args = task.instantiate(sample.knob_manager)
            except Exception as exc:  # a knob set the rules cannot replay
                out.append(MeasureResult((exc,), MeasureErrorNo.INSTANTIATION_ERROR, 0.0, 0.0))
                continue
            if self.measure_fn is not None:
                out.append(self.measure_fn(task, handle, args))
            else:
                out.append(measure_handle(task, handle, args, opt.number, opt.repeat, opt.min_repeat_ms,
                                          opt.flush_l2, getattr(task, "device_id", opt.device_id)))
        return out

    def run(self, samples, perf_buffer):
        if not samples:
            return
        task = samples[0].task
        for sample in samples:
            assert task.name == sample.task.name
        res = self.results2tup(self.measure_batch(samples))
        for sample, (error, perf) in zip(samples, res):
            sample.perf = perf
            sample.valid = error == 0
            perf_buffer.record(sample)
        if getattr(task.config, "verbose", False):
            print("TASK %s, Cur best %f" % (task.name, perf_buffer.best_perf))
