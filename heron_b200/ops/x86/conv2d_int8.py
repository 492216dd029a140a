"""The DL Boost NHWC conv (ops/x86/conv2d_int8.py:31-109): uint8 input, packed int8 filter."""
from ..cuda.conv2d import conv_out_extent
from ..spec import compute, placeholder, tcgen05_atom


def heron_conv2d_nhwc(ctx, N, H, W, CI, CO, KH, KW, stride, padding, dilation, w_format, in_dtype,
                      out_dtype):
    """Filter (CO/sco, KH, KW, CI/4, sco, 4); output (N, HO, WO, CO/sco, sco), i.e. NHWC."""
    assert w_format in ["OhwI64o4i", "OhwI48o4i", "OhwI32o4i"]
    split_co = int(w_format.split("I")[1].split("o")[0])
    split_ci = int(w_format.split("o")[1].split("i")[0])
    if isinstance(stride, int):
        stride_h = stride_w = stride
    else:
        stride_h, stride_w = stride
    if isinstance(dilation, int):
        dilation_h = dilation_w = dilation
    else:
        dilation_h, dilation_w = dilation
    assert isinstance(padding, int)
    Input = placeholder((N, H, W, CI), name="input", dtype="uint8")
    Filter = placeholder((CO // split_co, KH, KW, CI // split_ci, split_co, split_ci),
                         name="filter", dtype="int8")
    out_height = conv_out_extent(H, KH, stride_h, padding, dilation_h)
    out_width = conv_out_extent(W, KW, stride_w, padding, dilation_w)
    out = compute((N, out_height, out_width, CO // split_co, split_co), "int32", "conv",
                  "conv2d_nhwc_packed", [Input, Filter],
                  dict(N=N, H=H, W=W, CI=CI, CO=CO, KH=KH, KW=KW, stride=(stride_h, stride_w),
                       padding=padding, dilation=(dilation_h, dilation_w), sco=split_co,
                       in_dtype="uint8", out_dtype="int32"))
    info = {
        "name": "x86_dot",
        "stage_orgination": [("conv", "addCacheWriteGlobal")],
        "com": ("conv.global", (4, 3)),
        "intrin": [tcgen05_atom("uint8", "int32"), 16, 4],
    }
    ctx.set_info(info)
    ctx.set_axis_map({
        "pad": ["s_0", "s_1", "s_2", "r_2"],
        "conv.global": ["s_0", "s_1", "s_2", "s_3", "s_4"],
    })
    return [out]
