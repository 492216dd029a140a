"""Dilated NHWC conv2d with the reference's signature (ops/cuda/dil.py:9-105).

The reference registers the dilated convolution as an operator of its own ("dil") whose compute
is the NHWC tensor-core conv with `dilation > 1`: one dilation for both axes, integer padding on
all four sides, the same (N, CI, CO) shape rule, the same tensorize hints.  The kernel family
takes the dilation as plain conv geometry, so the operator is the NHWC conv under its own name.
"""
from .conv2d import heron_conv2d_nhwc_tensorcore


def heron_dil_tensorcore(ctx, N, H, W, CI, CO, KH, KW, stride, padding, dilation, in_dtype,
                         out_dtype):
    """out[n,y,x,f] = sum_{ry,rx,rc} Pad(in)[n, y*s+ry*d, x*s+rx*d, rc] * filter[ry,rx,rc,f]
    (ops/cuda/dil.py:47-66); output extent from the dilated kernel size (ops/cuda/dil.py:38-45)."""
    return heron_conv2d_nhwc_tensorcore(ctx, N, H, W, CI, CO, KH, KW, stride, padding, dilation,
                                        in_dtype, out_dtype)
