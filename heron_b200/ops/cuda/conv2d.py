"""NHWC conv2d with the reference's signature (ops/cuda/conv2d.py:137-232)."""
from ..spec import compute, placeholder, tcgen05_atom


def conv_out_extent(size, k, stride, pad, dilation):
    """(size - dilated_k + pad_before + pad_after) // stride + 1 (ops/cuda/conv2d.py:165-175)."""
    return (size - ((k - 1) * dilation + 1) + 2 * pad) // stride + 1


def heron_conv2d_nhwc_tensorcore(ctx, N, H, W, CI, CO, KH, KW, stride, padding, dilation, in_dtype,
                                 out_dtype):
    """out[n,y,x,f] = sum_{ry,rx,rc} Pad(in)[n, y*s+ry*d, x*s+rx*d, rc] * filter[ry,rx,rc,f]."""
    assert isinstance(stride, int) or len(stride) == 2
    assert isinstance(dilation, int) or len(dilation) == 2
    if isinstance(stride, int):
        stride_h = stride_w = stride
    else:
        stride_h, stride_w = stride
    # The reference keeps one dilation for both axes (ops/cuda/conv2d.py:149-152).
    if not isinstance(dilation, int):
        dilation = dilation[1]
    assert isinstance(padding, int), "integer padding: the same amount on all four sides"
    # Shape rule of the reference (ops/cuda/conv2d.py:158-165), kept so that a case the
    # reference rejects is rejected here too.
    assert (
        (N % 16 == 0 and CI % 16 == 0 and CO % 16 == 0)
        or (N % 8 == 0 and CI % 16 == 0 and CO % 32 == 0)
        or (N % 32 == 0 and CI % 16 == 0 and CO % 8 == 0)
    ), "The shape of (N, CI, CO) must be multiple of (16, 16, 16) or (32, 16, 8) or (8, 16, 32) for now"
    Input = placeholder((N, H, W, CI), name="input", dtype=in_dtype)
    Filter = placeholder((KH, KW, CI, CO), name="filter", dtype=in_dtype)
    H_O = conv_out_extent(H, KH, stride_h, padding, dilation)
    W_O = conv_out_extent(W, KW, stride_w, padding, dilation)
    Output = compute((N, H_O, W_O, CO), out_dtype, "out", "conv2d_nhwc", [Input, Filter],
                     dict(N=N, H=H, W=W, CI=CI, CO=CO, KH=KH, KW=KW, stride=(stride_h, stride_w),
                          padding=padding, dilation=(dilation, dilation), in_dtype=in_dtype,
                          out_dtype=out_dtype),
                     tag="conv2d_nhwc_tensorcore")
    info = {
        "name": "tensorcore",
        "stage_name": Output.op.name,
        "loadA": ("PaddedInput", (0, 3), "row_major", in_dtype),
        "loadB": (Filter.name, (2, 3), "row_major", in_dtype),
        "com": ((0, 2, 3), out_dtype),
        "store": ((0, 3), out_dtype),
        "compute_func": tcgen05_atom(in_dtype, out_dtype),
    }
    ctx.set_info(info)
    axis_map = {
        "PaddedInput.shared": ["s_0", "s_1", "s_2", "r_2"],
        "PaddedInput.shared.wmma.matrix_a": ["s_0", "s_1", "s_2", "r_2"],
        "filter.shared": ["r_0", "r_1", "r_2", "s_3"],
        "filter.shared.wmma.matrix_b": ["r_0", "r_1", "r_2", "s_3"],
        "out.wmma.accumulator.shared": ["s_0", "s_1", "s_2", "s_3"],
        "out.wmma.accumulator": ["s_0", "s_1", "s_2", "s_3"],
    }
    ctx.set_axis_map(axis_map)
    return [Output]


def heron_conv2d_nchw_tensorcore(ctx, N, H, W, CI, CO, KH, KW, stride, padding, dilation, in_dtype,
                                 out_dtype):
    """NCHW conv with the reference's signature (ops/cuda/conv2d.py:9-135): input (N,CI,H,W),
    filter (CO,CI,KH,KW), output (N,CO,HO,WO).  The reference pads a 3-channel filter by one zero
    tap per axis and the input by one more row and column; that changes neither the output extent
    nor any value, so it is not reproduced."""
    assert dilation == 1
    assert isinstance(stride, int) or len(stride) == 2
    if isinstance(stride, int):
        stride_h = stride_w = stride
    else:
        stride_h, stride_w = stride
    assert isinstance(padding, int)
    if CI == 3:
        assert KH == 3 or KH == 7
        assert KW == 3 or KW == 7
    else:
        assert CI % 16 == 0
    Input = placeholder((N, CI, H, W), name="input", dtype=in_dtype)
    Filter = placeholder((CO, CI, KH, KW), name="filter", dtype=in_dtype)
    H_O = conv_out_extent(H, KH, stride_h, padding, 1)
    W_O = conv_out_extent(W, KW, stride_w, padding, 1)
    output = compute((N, CO, H_O, W_O), out_dtype, "output", "conv2d_nchw", [Input, Filter],
                     dict(N=N, H=H, W=W, CI=CI, CO=CO, KH=KH, KW=KW, stride=(stride_h, stride_w),
                          padding=padding, dilation=(1, 1), in_dtype=in_dtype, out_dtype=out_dtype),
                     tag="default, stride:%d" % (H_O * W_O))
    # The reference multiplies B (filter, CO x K) by A (im2col, pixels x K): its "loadA" is the filter.
    info = {
        "name": "tensorcore",
        "stage_name": "C",
        "loadA": ("B", (0, 1), "row_major", in_dtype),
        "loadB": ("A", (0, 1), "col_major", in_dtype),
        "com": ((0, 0, 1), out_dtype),
        "store": ((0, 1), out_dtype),
        "compute_func": tcgen05_atom(in_dtype, out_dtype),
    }
    ctx.set_info(info)
    ctx.set_axis_map({
        "B.shared": ["s_0", "r_0"],
        "B.shared.wmma.matrix_a": ["s_0", "r_0"],
        "A.shared": ["s_1", "r_0"],
        "A.shared.wmma.matrix_b": ["s_1", "r_0"],
        "C.wmma.accumulator.shared": ["s_0", "s_1"],
        "C.wmma.accumulator": ["s_0", "s_1"],
    })
    return [output]
