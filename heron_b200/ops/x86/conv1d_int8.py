"""The DL Boost NWC conv1d (ops/x86/conv1d_int8.py:31-101): uint8 input, packed int8 filter."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_conv1d_nwc(ctx, batch, in_width, co, ci, kernel, stride, padding, dilation, w_format,
                     in_dtype, out_dtype):
    """Input (batch, W, ci); filter (co/sco, kernel, ci/4, sco, 4); output (batch, W_O, co/sco, sco).
    Note the argument order of the reference: output channels come before input channels."""
    assert w_format in ["OwI64o4i", "OwI48o4i", "OwI32o4i"]
    split_co = int(w_format.split("I")[1].split("o")[0])
    split_ci = int(w_format.split("o")[1].split("i")[0])
    assert isinstance(stride, int) and isinstance(dilation, int) and isinstance(padding, int)
    Input = placeholder((batch, in_width, ci), name="input", dtype="uint8")
    Filter = placeholder((co // split_co, kernel, ci // split_ci, split_co, split_ci), name="filter",
                         dtype="int8")
    out_width = (in_width - ((kernel - 1) * dilation + 1) + 2 * padding) // stride + 1
    out = compute((batch, out_width, co // split_co, split_co), "int32", "conv", "conv1d_nwc_packed",
                  [Input, Filter],
                  dict(N=batch, W=in_width, CI=ci, CO=co, KW=kernel, stride=stride, padding=padding,
                       dilation=dilation, sco=split_co, in_dtype="uint8", out_dtype="int32"))
    info = {
        "name": "x86_dot",
        "stage_orgination": [("conv", "addCacheWriteGlobal")],
        "com": ("conv.global", (3, 2)),
        "intrin": [tcgen05_atom("uint8", "int32"), 16, 4],
    }
    ctx.set_info(info)
    ctx.set_axis_map({
        "pad": ["s_0", "s_1", "r_1"],
        "conv.global": ["s_0", "s_1", "s_2", "s_3"],
    })
    return [out]
