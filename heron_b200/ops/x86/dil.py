"""Dilated DL Boost NHWC conv with the reference's signature (ops/x86/dil.py:30-107).

Same operator as the packed-filter NHWC conv (uint8 input, int8 filter in
(CO/sco, KH, KW, CI/4, sco, 4), int32 output ordered as NHWC) registered under "dil"; the
dilation may differ per axis (ops/x86/dil.py:43-46).
"""
from .conv2d_int8 import heron_conv2d_nhwc


def heron_dil_nhwc(ctx, N, H, W, CI, CO, KH, KW, stride, padding, dilation, w_format, in_dtype,
                   out_dtype):
    return heron_conv2d_nhwc(ctx, N, H, W, CI, CO, KH, KW, stride, padding, dilation, w_format,
                             in_dtype, out_dtype)
