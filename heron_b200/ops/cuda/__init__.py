"""The tensor-core operator registry (ops/cuda/__init__.py:15-32), limited to the hot path."""
from .batch_matmul import heron_batch_matmul
from .conv2d import heron_conv2d_nchw_tensorcore, heron_conv2d_nhwc_tensorcore
from .dense import heron_dense

_OPMAP = {
    "gemm": heron_dense,
    "bmm": heron_batch_matmul,
    "c2d": heron_conv2d_nchw_tensorcore,
    "c2d_nhwc": heron_conv2d_nhwc_tensorcore,
}

# Names the reference registers that have no B200 kernel here.
_NOT_BUILT = ("gemv", "c1d", "c3d", "t2d", "mean", "var", "scan", "dil", "dep")


def getOpFromName(name):
    if name in _NOT_BUILT:
        raise NotImplementedError("operator %r is outside the GEMM / BMM / NHWC-conv hot path" % name)
    return _OPMAP[name]
