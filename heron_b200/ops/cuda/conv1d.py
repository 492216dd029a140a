"""NCW conv1d with the reference's signature (ops/cuda/conv1d.py:11-110)."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_conv1d_ncw_tensorcore(ctx, N, W, CI, CO, KW, stride, padding, dilation, in_dtype, out_dtype):
    """out[n,c,q] = sum_{ci,kw} Pad(in)[n, ci, q*stride + kw] * filter[c, ci, kw]; input (N,CI,W),
    filter (CO,CI,KW), output (N,CO,W_O).  The reference writes it as an explicit im2col GEMM
    C[CO, N*W_O] = B[CO, CI*KW] . A[N*W_O, CI*KW]^T (ops/cuda/conv1d.py:33-69); the sum is the same."""
    assert isinstance(stride, int)
    assert dilation == 1  # ops/cuda/conv1d.py:16
    assert isinstance(padding, int)
    Input = placeholder((N, CI, W), name="input", dtype=in_dtype)
    Filter = placeholder((CO, CI, KW), name="filter", dtype=in_dtype)
    W_O = (W - KW + 2 * padding) // stride + 1
    output = compute((N, CO, W_O), out_dtype, "output", "conv1d_ncw", [Input, Filter],
                     dict(N=N, W=W, CI=CI, CO=CO, KW=KW, stride=stride, padding=padding,
                          in_dtype=in_dtype, out_dtype=out_dtype), tag="default")
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
