"""The reference's "transposed" DL Boost conv (ops/x86/t2d.py:59-135), stride 1.

As in the tensor-core form, the operator is a correlation of the zero-expanded input, padded by
(K-1)*dilation - padding zeros, with the packed filter as stored; for stride 1 that is the packed
NHWC conv with that padding.  For stride > 1 the reference indexes its expanded tensor at
y*stride + ry*dilation (t2d.py:102-106), past its end, so those cases are refused.
"""
from .conv2d_int8 import heron_conv2d_nhwc


def heron_conv2d_transposed_nhwc(ctx, N, H, W, CI, CO, KH, KW, stride, padding, dilation, outpadding,
                                 w_format, in_dtype, out_dtype):
    assert isinstance(padding, int) and isinstance(dilation, int)
    if stride != 1 and stride != (1, 1):
        raise NotImplementedError("t2d with stride %s: the reference's expression reads past the end of its "
                                  "expanded, padded input (t2d.py:102-106)" % (stride,))
    assert outpadding == 0
    assert KH == KW, "one padding value for both axes"
    pad = (KH - 1) * dilation - padding
    assert pad >= 0
    return heron_conv2d_nhwc(ctx, N, H, W, CI, CO, KH, KW, 1, pad, dilation, w_format, in_dtype, out_dtype)
