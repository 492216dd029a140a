"""NCDHW conv3d with the reference's signature (ops/cuda/conv3d.py:9-125)."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_conv3d_ncdhw_tensorcore(ctx, N, D, H, W, CI, CO, KD, KH, KW, stride, padding, dilation, in_dtype,
                                  out_dtype):
    """Input (N,CI,D,H,W), filter (CO,CI,KD,KH,KW), output (N,CO,D_O,H_O,W_O):
    out[n,c,d,p,q] = sum_{ci,kd,kh,kw} Pad(in)[n,ci,d*sd+kd,p*sh+kh,q*sw+kw] * filter[c,ci,kd,kh,kw].
    The reference writes it as an explicit im2col GEMM C[CO, N*D_O*H_O*W_O] = B . A^T
    (ops/cuda/conv3d.py:37-75); the sum is the same."""
    assert dilation == 1  # ops/cuda/conv3d.py:14
    assert isinstance(stride, int) or len(stride) == 3
    if isinstance(stride, int):
        stride_d = stride_h = stride_w = stride
    else:
        stride_d, stride_h, stride_w = stride
    assert isinstance(padding, int)
    Input = placeholder((N, CI, D, H, W), name="input", dtype=in_dtype)
    Filter = placeholder((CO, CI, KD, KH, KW), name="filter", dtype=in_dtype)
    D_O = (D - KD + 2 * padding) // stride_d + 1
    H_O = (H - KH + 2 * padding) // stride_h + 1
    W_O = (W - KW + 2 * padding) // stride_w + 1
    output = compute((N, CO, D_O, H_O, W_O), out_dtype, "output", "conv3d_ncdhw", [Input, Filter],
                     dict(N=N, D=D, H=H, W=W, CI=CI, CO=CO, KD=KD, KH=KH, KW=KW,
                          stride=(stride_d, stride_h, stride_w), padding=padding, in_dtype=in_dtype,
                          out_dtype=out_dtype), tag="default")
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
