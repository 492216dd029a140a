"""The reference's "transposed" NCHW conv (ops/cuda/conv2d_transposed.py:59-171), stride 1.

What the reference computes is a plain correlation of the zero-expanded, zero-padded input with
the filter as stored (no flip, no channel swap):
    out[n,c,p,q] = sum_{ci,kh,kw} Pad(Expand(in))[n, ci, p*stride + kh, q*stride + kw] * w[c,ci,kh,kw]
with (K-1-padding) zeros before and (K-1-padding+outpadding) after each spatial axis
(conv2d_transposed.py:82-107).  For stride 1 the expansion is the identity and this is the NCHW
conv with padding K-1-padding, which is what runs here.

For stride > 1 the reference's expression is not well defined: the expanded, padded tensor has
(H-1)*stride + 1 + 2*(K-1-padding) + outpadding = H_O + K - 1 rows (lines 18-19, 84-92), while the
im2col stage indexes it at p*stride + kh for p < H_O (lines 100-107), i.e. up to stride*(H_O-1)+K-1,
beyond its end.  There is no result to reproduce, so those cases are refused.
"""
from .conv2d import heron_conv2d_nchw_tensorcore


def heron_conv2d_nchw_transposed_tensorcore(ctx, N, H, W, CI, CO, KH, KW, stride, padding, dilation,
                                            outpadding, in_dtype, out_dtype):
    assert isinstance(padding, int)
    assert isinstance(stride, int)
    assert isinstance(dilation, int)
    if stride != 1:
        raise NotImplementedError("t2d with stride %d: the reference's expression reads past the end of its "
                                  "expanded, padded input (conv2d_transposed.py:100-107)" % stride)
    # the reference applies the dilation to the output extent only (lines 79-83), not to the taps
    # (lines 100-107); with dilation 1 the two agree
    assert dilation == 1 and outpadding == 0
    assert KH == KW, "one padding value for both axes"
    assert KH - 1 - padding >= 0
    return heron_conv2d_nchw_tensorcore(ctx, N, H, W, CI, CO, KH, KW, 1, KH - 1 - padding, 1, in_dtype,
                                        out_dtype)
