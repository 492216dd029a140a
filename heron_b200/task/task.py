"""Task: an operator instance plus its knob space, with the reference's interface
(task/task.py:13-103).

``instantiate(knob_manager)`` is the drop-in boundary.  In the reference it returns
``(schedule, args)`` for ``tvm.build``; here it returns ``(KernelHandle, args)`` where the handle
launches the sm_100a kernel specialised by the solved knob values and ``args`` is the same list
of tensors — inputs in discovery order, then the output (task/task.py:81).
"""
import json
import os

from ..schedule.constraints import KnobManager
from ..schedule.context import KernelSchedule, buildContext
from ..schedule.sched_op import get_op_methods, sched_via_rule


class KernelHandle:
    """The built artefact: called with device tensors in ``args`` order (inputs..., output).

    Stands where the module returned by ``tvm.build(s, args)`` stands
    (tests/quick_start/dlboost/run.py:44-46).  ``plan(*tensors)`` binds it to fixed buffers for
    repeated launches, which is what the measurement code times.
    """

    # An immediate call on small tensors spends more time encoding its three tensor maps on the
    # host than the GPU spends on the problem.  Calls whose tensors total at most this many bytes
    # therefore keep their plan: a later call on the same buffers only launches it.
    SMALL_CALL_BYTES = 1 << 20
    PLAN_CACHE_SIZE = 16

    def __init__(self, op, knobs):
        self.op = op
        self.knobs = dict(knobs)
        self.entry_name = op.name
        self._small_plans = {}  # (data_ptr, shape, dtype, device) per tensor -> Plan, oldest first

    def _call(self, planned, *tensors):
        from .. import kernels as K
        kind, p = self.op.kind, self.op.params
        knobs = self.knobs or None
        if kind == "gemm":
            a, b, out = tensors
            fn = K.plan_gemm if planned else K.gemm
            return fn(a, b, out=out, knobs=knobs)
        if kind == "bmm":
            a, b, out = tensors
            fn = K.plan_bmm if planned else K.bmm
            return fn(a, b, out=out, knobs=knobs)
        if kind == "conv2d_nhwc":
            x, w, out = tensors
            fn = K.plan_conv2d_nhwc if planned else K.conv2d_nhwc
            return fn(x, w, stride=p["stride"], padding=p["padding"], dilation=p["dilation"], out=out,
                      knobs=knobs)
        if kind == "conv2d_nchw":
            x, w, out = tensors
            fn = K.plan_conv2d_nchw if planned else K.conv2d_nchw
            return fn(x, w, stride=p["stride"], padding=p["padding"], out=out, knobs=knobs)
        if kind == "conv2d_nhwc_packed":
            x, w, out = tensors
            fn = K.plan_conv2d_nhwc_packed if planned else K.conv2d_nhwc_packed
            return fn(x, w, p["CO"], p["KH"], p["KW"], stride=p["stride"], padding=p["padding"],
                      dilation=p["dilation"], sco=p["sco"], out=out, knobs=knobs)
        if kind == "conv3d_ncdhw":
            x, w, out = tensors
            fn = K.plan_conv3d_ncdhw if planned else K.conv3d_ncdhw
            return fn(x, w, stride=p["stride"], padding=p["padding"], out=out, knobs=knobs)
        if kind == "scan":
            a, out = tensors
            fn = K.plan_scan if planned else K.scan
            return fn(a, p["N"], out=out, knobs=knobs)
        if kind == "gemv":
            a, x, out = tensors
            fn = K.plan_gemv if planned else K.gemv
            return fn(a, x, out=out, knobs=knobs)
        if kind == "conv1d_ncw":
            x, w, out = tensors
            fn = K.plan_conv1d_ncw if planned else K.conv1d_ncw
            return fn(x, w, stride=p["stride"], padding=p["padding"], out=out, knobs=knobs)
        if kind == "conv1d_nwc_packed":
            x, w, out = tensors
            fn = K.plan_conv1d_nwc_packed if planned else K.conv1d_nwc_packed
            return fn(x, w, p["CO"], p["KW"], stride=p["stride"], padding=p["padding"],
                      dilation=p["dilation"], sco=p["sco"], out=out, knobs=knobs)
        raise NotImplementedError(kind)

    def __call__(self, *tensors):
        nbytes = sum(t.numel() * t.element_size() for t in tensors)
        if nbytes > self.SMALL_CALL_BYTES:
            return self._call(False, *tensors)
        # (a cached plan holds references to its tensors, so an address in a key cannot be handed
        # to another tensor while the entry lives)
        key = tuple((t.data_ptr(), tuple(t.shape), t.dtype, t.device) for t in tensors)
        plan = self._small_plans.pop(key, None)
        if plan is None:
            plan = self._call(True, *tensors)
            while len(self._small_plans) >= self.PLAN_CACHE_SIZE:
                self._small_plans.pop(next(iter(self._small_plans))).close()
        self._small_plans[key] = plan  # most recently used last
        return plan.launch()

    def plan(self, *tensors):
        return self._call(True, *tensors)


class Task:
    def __init__(self, name, opfunc, args, target, target_host=None):
        self.name = name
        self.args = args
        self.opfunc = opfunc
        self.target = target
        self.target_host = target_host
        self.build_kwargs = None
        self.knob_manager = KnobManager()
        self.not_verify_correctness = True
        self.ref_input = None
        self.ref_output = None
        self.config = None
        self.sched_desc = ""

    def code(self):
        return self.name

    def _codegen_type(self):
        return self.config.codegen_type if self.config is not None else "GPU_TENSOR_CORE"

    def apply_best(self, path):
        """Loads the best record of a ``records.txt`` and instantiates it (task/task.py:30-43)."""
        if self.knob_manager.sched_tups == []:
            self.make_stage_schedules()
        to_sort = []
        for row in open(path):
            json_dict = json.loads(row)
            to_sort.append((json_dict["perf"], json_dict["param"]))
        sorted_pairs = sorted(to_sort, key=lambda x: -x[0])
        self.knob_manager.solved_knob_vals_phenotype = sorted_pairs[0][1]
        self.knob_manager.runtime_perf = sorted_pairs[0][0]
        self.knob_manager.is_building = False
        return self.instantiate(self.knob_manager)

    def apply_sample(self, sample):
        self.knob_manager.solved_knob_vals_phenotype = dict(sample.knob_manager.solved_knob_vals_phenotype)
        self.knob_manager.runtime_perf = sample.perf
        self.knob_manager.is_building = False
        return self.instantiate(self.knob_manager)

    def getOut(self):
        ctx = buildContext(self._codegen_type(), self.knob_manager, self.build_kwargs, str(self.target))
        return self.opfunc(ctx, *self.args)

    def make_stage_schedules(self):
        """Builds the knob space: runs the operator function, applies the schedule rules (which
        register knobs and constraints), and checks that the space is not empty
        (task/task.py:56-68)."""
        ctx = buildContext(self._codegen_type(), self.knob_manager, self.build_kwargs, str(self.target))
        outs = self.opfunc(ctx, *self.args)
        s = KernelSchedule(outs)
        ctx.init_tensor_dict(outs)
        sched_via_rule(self._codegen_type(), ctx, s)
        self.sched_desc = ctx.sched_desc
        self.knob_manager.is_building = False
        valid, _ = self.knob_manager.solver.solve({}, {})
        self.dump_constraints()
        assert valid

    def dump_constraints(self):
        if self.config is None or not getattr(self.config, "log_dir", None):
            return
        if not os.path.isdir(self.config.log_dir):
            return
        with open(os.path.join(self.config.log_dir, "constraints.py"), "w") as f:
            f.write(self.knob_manager.solver.dump())

    def instantiate(self, knob_manager):
        """Knob values -> launchable kernel (task/task.py:76-89): replays the recorded rules so
        that each reads its solved values, then wraps them in a KernelHandle."""
        ctx = buildContext(self._codegen_type(), knob_manager, self.build_kwargs, str(self.target))
        outs = self.opfunc(ctx, *self.args)
        s = KernelSchedule(outs)
        ctx.init_tensor_dict(outs)
        args = ctx.input_tensors + outs
        op_methods = get_op_methods(self._codegen_type())
        for act_name, stage_name in knob_manager.sched_tups:
            op_methods[act_name](act_name).perform(s, stage_name, ctx)
        ctx.pos_process(s)
        knob_manager.sched_desc = ctx.sched_desc
        knobs = {k: v for k, v in ctx.kernel_knobs.items() if v is not None}
        return KernelHandle(outs[0].op, knobs), args

    def set_verify_func(self, func, rtol=0.1):
        """``func(args) -> (inputs, expected_output)`` as numpy arrays; measured candidates whose
        output is not ``allclose`` to it are scored as wrong (task/task.py:91-96,
        runner/measure_methods.py:172-177)."""
        self.rtol = rtol
        self.not_verify_correctness = False
        self.ref_input, self.ref_output = func(self.args)

    def getStmt(self, knob_manager):
        """Text description of the instantiated kernel (the reference returns lowered TIR)."""
        handle, args = self.instantiate(knob_manager)
        return "%s%s knobs=%s" % (knob_manager.sched_desc, handle.op, sorted(handle.knobs.items()))
