"""Per-target state while a kernel configuration is being described
(schedule/context/context.py:7-90 and cuda_context.py / cpu_context.py of the reference).

The reference's contexts track TVM stages, tile structures and compute-at positions.  The B200
kernels are written by hand, so the context tracks instead: the operator (from the tensors the
operator function returned), the hints it passed (`info`, `axis_map`), the hardware limits the
constraints refer to, and `kernel_knobs` — the tile / stage / swizzle values the schedule rules
read back from the knob manager once a point is chosen.
"""

# Limits of one B200 SM the constraint model refers to.
B200_LIMITS = {
    "max_shared_memory_per_block": 232448,  # 227 KiB opt-in dynamic shared memory
    "tmem_columns": 512,
    "tile_m": 128,
    "max_stages": 12,
    "epilogue_staging_bytes": 4 * 2 * 4096,
    "smem_slack_bytes": 2048 + 512,
    "sm_count": 148,
}


class KernelSchedule:
    """What takes the place of ``te.create_schedule(...)``: the operator outputs being scheduled."""

    def __init__(self, outs):
        self.outputs = list(outs)
        self.stages = [o.op for o in outs]


class Context:
    def __init__(self, knob_manager, build_kwargs, target_name):
        self.sched_desc = ""
        self.codegen_type = None
        self.target_name = target_name
        self.build_kwargs = build_kwargs or {}
        self.tensor_dict = {}
        self.input_tensors = []
        self.tensorize_info = None
        self.axis_map = {}
        self.knob_manager = knob_manager
        self.limits = dict(B200_LIMITS)
        self.limits.update(self.build_kwargs.get("limits", {}))
        self.kernel_knobs = {}

    def set_info(self, info):
        self.tensorize_info = info

    def set_axis_map(self, axis_map):
        self.axis_map = axis_map

    def init_tensor_dict(self, outs):
        """Collects the placeholders in discovery order, as the reference does (context.py:38-48):
        the built kernel's arguments are ``input_tensors + outs``."""
        if len(outs) == 0:
            return
        inputs = []
        for tensor in outs:
            self.tensor_dict[tensor.name] = tensor
            input_tensors = tensor.op.input_tensors
            inputs += input_tensors
            if len(input_tensors) == 0 and tensor not in self.input_tensors:
                self.input_tensors.append(tensor)
        self.init_tensor_dict(inputs)

    def addSchedDesc(self, strs, add2Solver=False):
        self.sched_desc += strs

    def addSched(self, op_name, stage_name, s):
        from ..sched_op import get_op_methods
        self.knob_manager.sched_tups.append((op_name, stage_name))
        get_op_methods(self.codegen_type)[op_name](op_name).perform(s, stage_name, self)

    def pos_process(self, s):
        pass


class TENSORCOREContext(Context):
    """The tensor-core target (cuda_context.py:93-108): operators from ops/cuda."""

    def __init__(self, knob_manager, build_kwargs, target_name):
        Context.__init__(self, knob_manager, build_kwargs, target_name)
        self.codegen_type = "GPU_TENSOR_CORE"
        self.is_tensorcore = True

    def set_info(self, info):
        if info is None:
            return
        assert info["name"] == "tensorcore"
        self.tensorize_info = info


class CPUContext(Context):
    """The DL Boost target (cpu_context.py:8-34): operators from ops/x86, here run on the B200's
    int8 tensor path with the x86 operators' dtypes and layouts."""

    def __init__(self, knob_manager, build_kwargs, target_name):
        Context.__init__(self, knob_manager, build_kwargs, target_name)
        self.codegen_type = "CPU"

    def set_info(self, info):
        if info is None:
            return
        assert info["name"] == "x86_dot"
        self.tensorize_info = info
