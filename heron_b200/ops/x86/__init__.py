"""The DL Boost operator registry (ops/x86/__init__.py:11-23), limited to the hot path."""
from .batch_matmul import heron_batch_matmul
from .conv1d_int8 import heron_conv1d_nwc
from .conv2d_int8 import heron_conv2d_nhwc
from .dense import heron_dense
from .dil import heron_dil_nhwc
from .gemv import heron_gemv
from .scan import heron_scan
from .t2d import heron_conv2d_transposed_nhwc

_OPMAP = {
    "gemm": heron_dense,
    "gemv": heron_gemv,
    "c1d": heron_conv1d_nwc,
    "bmm": heron_batch_matmul,
    "c2d": heron_conv2d_nhwc,
    "dil": heron_dil_nhwc,
    "scan": heron_scan,
    "t2d": heron_conv2d_transposed_nhwc,
}

_NOT_BUILT = ("c3d",)


def getOpFromName(name):
    if name in _NOT_BUILT:
        raise NotImplementedError("operator %r is outside the GEMM / BMM / conv hot path and its neighbours" % name)
    return _OPMAP[name]
