"""Store of measured samples and writer of ``records.txt`` (perf/perfBuffer.py:7-56 of the
reference).  One JSON object per line with the reference's fields — ``code``, ``perf``,
``latency``, ``time``, ``param`` — so that records written here can be read by the reference's
``Task.apply_best`` (task/task.py:30-43) and the other way round."""
import json
import math
import os
import time


class perfBuffer:
    def __init__(self, config):
        self.perfs = {}
        self.data_x = []
        self.data_y = []
        self.samples = []
        self.measured_keys = []
        self.best_perf = None
        self.best_sample = None
        self.config = config

    def record(self, sample):
        code = sample.stmt_code
        if code in self.perfs:
            return
        self.measured_keys.append(code)
        self.perfs[code] = sample.perf
        if sample.perf != 0:
            self.samples.append(sample)
            self.data_x.append(sample.point)
            self.data_y.append(sample.perf)
        if self.best_perf is None or sample.perf > self.best_perf:
            self.best_perf = sample.perf
            self.best_sample = sample
        log_dir = getattr(self.config, "log_dir", None)
        if log_dir and os.path.isdir(log_dir):
            with open(os.path.join(log_dir, "records.txt"), "a") as f:
                f.write(self.encode(sample) + "\n")

    def encode(self, sample):
        return json.dumps({
            "code": sample.stmt_code,
            "perf": sample.perf,
            "latency": math.exp(-sample.perf),
            "time": time.time(),
            "param": sample.knob_manager.solved_knob_vals_phenotype,
        })

    def getPerf(self, task):
        code = task.stmt_code
        if code not in self.perfs:
            return None
        return self.perfs[code]


def warm_start(perf_buffer, task, path):
    """Reads an existing ``records.txt`` back into a buffer (the reference can only re-apply the
    best record; its tuning runs start from an emptied directory, environment.py:19-22)."""
    from ..sample import Sample
    n = 0
    for row in open(path):
        d = json.loads(row)
        s = Sample(task)
        s.fromCode(d["code"])
        s.knob_manager.solved_knob_vals_phenotype = dict(d["param"])
        s.perf = d["perf"]
        s.predict = d["perf"]
        s.valid = d["perf"] != 0
        code = s.stmt_code
        if code in perf_buffer.perfs:
            continue
        perf_buffer.measured_keys.append(code)
        perf_buffer.perfs[code] = s.perf
        if s.perf != 0:
            perf_buffer.samples.append(s)
            perf_buffer.data_x.append(s.point)
            perf_buffer.data_y.append(s.perf)
        if perf_buffer.best_perf is None or s.perf > perf_buffer.best_perf:
            perf_buffer.best_perf, perf_buffer.best_sample = s.perf, s
        n += 1
    return n
