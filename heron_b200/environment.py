"""Env: owns the task, the tuner, the runner and the measured-sample store
(environment.py:10-108 of the reference)."""
import os
import shutil
import time

from .perf.perfBuffer import perfBuffer
from .runner.runner import Runner
from .schedule.context import B200_LIMITS
from .schedule.sched_op import get_op_methods
from .task.task import Task
from .tuner import (CGATuner, ConstrainedRandomWalkerSATuner, CRandTuner, GATuner, IDEATuner, RandomWalkSATuner,
                    RCGATuner, SDGATuner, SRGATuner)
from .utils import mkdir

_TUNERS = {
    "CRAND": CRandTuner,
    "CGA": CGATuner,
    "RCGA": RCGATuner,
    "GA": GATuner,
    "SDGA": SDGATuner,
    "SRGA": SRGATuner,
    "IDEA": IDEATuner,
    "SA": RandomWalkSATuner,
    "CSA": ConstrainedRandomWalkerSATuner,
}


class Env:
    def __init__(self, measure_option, config, measure_fn=None):
        self.config = config
        self.runner = Runner(measure_option, measure_fn)
        self.num_ops = len(get_op_methods(config.codegen_type))
        self.build_kwargs = None
        self.task = None

    def init_dir(self):
        if os.path.exists(self.config.log_dir):
            shutil.rmtree(self.config.log_dir)
        mkdir(self.config.log_dir)

    def get_build_kwargs(self, task):
        # The reference asks TVM for the GPU's limits (threads, shared memory); the constraint
        # model here refers to the B200's SM limits.
        limits = dict(B200_LIMITS)
        try:  # prefer the numbers the built library reports over the table in the package
            from . import _lib
            limits.update(_lib.kernel_limits())
        except ImportError:
            pass
        self.build_kwargs = {"limits": limits}

    def tune(self, task_name, pretrained=False):
        self.init_dir()
        start = time.time()
        self.task.make_stage_schedules()
        self.dump_schedule()
        res = self.tuner.run(self)
        if self.config.verbose:
            print("Heron tune time spent ", time.time() - start)
        return res

    def dump_schedule(self):
        with open(os.path.join(self.config.log_dir, "schedule.py"), "w") as f:
            f.write(self.task.sched_desc)

    def createTask(self, name, opfunc, args, target, target_host=None, dump_const_desc=False):
        assert self.task is None
        self.config.task_name = name
        task = Task(name, opfunc, args, target, target_host)
        task.knob_manager.dump_descs = dump_const_desc
        if self.build_kwargs is None:
            self.get_build_kwargs(task)
        task.build_kwargs = self.build_kwargs
        task.config = self.config
        self.task = task
        self.config.setEnv(self)
        try:
            self.tuner = _TUNERS[self.config.opt_method](self.config)
        except KeyError:
            raise ValueError("Unsupportted opt method")
        if self.config.use_cost_model:
            self.tuner.buildCostModel(self.task)
        self.perf_buffer = perfBuffer(self.config)
        return task

    def evalSamples(self, samples):
        self.runner.run(samples, self.perf_buffer)
        return samples
