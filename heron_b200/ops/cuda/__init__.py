"""The tensor-core operator registry (ops/cuda/__init__.py:15-32): the hot path (gemm, bmm, c2d_nhwc)
and the operators next to it that run on the same kernels (c2d, c3d, dil, c1d, gemv, scan, t2d at stride 1)."""
from .batch_matmul import heron_batch_matmul
from .conv1d import heron_conv1d_ncw_tensorcore
from .conv3d import heron_conv3d_ncdhw_tensorcore
from .conv2d_transposed import heron_conv2d_nchw_transposed_tensorcore
from .conv2d import heron_conv2d_nchw_tensorcore, heron_conv2d_nhwc_tensorcore
from .dense import heron_dense
from .dil import heron_dil_tensorcore
from .gemv import heron_gemv
from .scan import heron_scan

_OPMAP = {
    "gemv": heron_gemv,
    "gemm": heron_dense,
    "c1d": heron_conv1d_ncw_tensorcore,
    "c3d": heron_conv3d_ncdhw_tensorcore,
    "bmm": heron_batch_matmul,
    "c2d": heron_conv2d_nchw_tensorcore,
    "c2d_nhwc": heron_conv2d_nhwc_tensorcore,
    "dil": heron_dil_tensorcore,
    "scan": heron_scan,
    "t2d": heron_conv2d_nchw_transposed_tensorcore,
}

# Names the reference registers that have no B200 kernel here.
_NOT_BUILT = ("mean", "var", "dep")


def getOpFromName(name):
    if name in _NOT_BUILT:
        raise NotImplementedError("operator %r is outside the GEMM / BMM / conv hot path and its neighbours" % name)
    return _OPMAP[name]
