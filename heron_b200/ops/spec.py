"""Shape-and-dtype descriptions that stand where the reference's ``te.Tensor`` / ``te.compute`` stand.

The reference's operator functions build TVM tensor expressions and return ``[out]``
(ops/cuda/dense.py:4-17); callers then read ``tensor.shape``, ``tensor.dtype``, ``tensor.name``
and ``tensor.op.input_tensors`` (schedule/context/context.py:38-48,
tests/quick_start/dlboost/run.py:52-58).  ``TensorSpec`` and ``OpSpec`` carry exactly those
attributes, plus the operator kind and parameters the B200 kernels are launched from.
"""


class OpSpec:
    """The producing operation of a tensor: a placeholder (no inputs) or one of gemm/bmm/conv."""

    def __init__(self, name, kind, input_tensors=(), params=None, tag=""):
        self.name = name
        self.kind = kind  # 'placeholder', 'gemm', 'bmm', 'conv2d_nhwc', 'conv2d_nhwc_packed'
        self.input_tensors = list(input_tensors)
        self.params = dict(params or {})
        self.tag = tag

    def __repr__(self):
        return "OpSpec(%s:%s)" % (self.kind, self.name)


class TensorSpec:
    def __init__(self, shape, dtype, name, op=None):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype
        self.name = name
        self.op = op if op is not None else OpSpec(name, "placeholder")

    @property
    def ndim(self):
        return len(self.shape)

    def __repr__(self):
        return "TensorSpec(%s, %s, %s)" % (self.name, self.shape, self.dtype)


def placeholder(shape, name, dtype):
    """Counterpart of ``te.placeholder(shape, name=..., dtype=...)``."""
    return TensorSpec(shape, dtype, name)


def compute(shape, dtype, name, kind, inputs, params, tag=""):
    """Counterpart of ``te.compute``: the output tensor of an operator on the hot path."""
    return TensorSpec(shape, dtype, name, OpSpec(name, kind, inputs, params, tag))


# MMA atom of the B200 kernels, handed to the context where the reference hands its wmma
# compute function (`compute_func` in the `info` dict, ops/cuda/dense.py:19-33): per instruction
# a 128 x N x (32 bytes of K) product accumulated in TMEM.
def tcgen05_atom(in_dtype, out_dtype):
    ebytes = {"float16": 2, "int8": 1, "uint8": 1}[in_dtype]
    return {
        "instruction": "tcgen05.mma.cta_group::1.kind::%s" % ("f16" if ebytes == 2 else "i8"),
        "m": 128,
        "n_step": 16,
        "n_max": 256,
        "k": 32 // ebytes,
        "accumulator": "float32" if ebytes == 2 else "int32",
        "out_dtype": out_dtype,
    }
