"""The DL Boost operator registry (ops/x86/__init__.py:11-23), limited to the hot path."""
from .batch_matmul import heron_batch_matmul
from .conv2d_int8 import heron_conv2d_nhwc
from .dense import heron_dense

_OPMAP = {
    "gemm": heron_dense,
    "bmm": heron_batch_matmul,
    "c2d": heron_conv2d_nhwc,
}

_NOT_BUILT = ("gemv", "c1d", "c3d", "dil", "t2d", "scan")


def getOpFromName(name):
    if name in _NOT_BUILT:
        raise NotImplementedError("operator %r is outside the GEMM / BMM / NHWC-conv hot path" % name)
    return _OPMAP[name]
