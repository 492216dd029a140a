from .context import B200_LIMITS, Context, CPUContext, KernelSchedule, TENSORCOREContext


def buildContext(_type, knob_manager, build_kwargs, target_name):
    """schedule/context/__init__.py:5-15 of the reference, for the two targets on the hot path."""
    if _type == "GPU_TENSOR_CORE":
        return TENSORCOREContext(knob_manager, build_kwargs, target_name)
    if _type == "CPU":
        return CPUContext(knob_manager, build_kwargs, target_name)
    raise ValueError("Unsupportted code gen type %s" % _type)
