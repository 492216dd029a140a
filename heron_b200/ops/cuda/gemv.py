"""Matrix-vector product in the reference's tensor-core form (ops/cuda/gemv.py:4-65)."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_gemv(ctx, M, K, in_dtype, out_dtype):
    """A (M,K), B (1,K), out (M,8): out[i,j] = sum_k A[i,k] * BPad[j,k] where BPad is B followed by
    seven rows of zeros (ops/cuda/gemv.py:12-30), so column 0 is the product and the rest is 0."""
    A = placeholder((M, K), name="A", dtype=in_dtype)
    B = placeholder((1, K), name="B", dtype=in_dtype)
    out = compute((M, 8), out_dtype, "dense", "gemv", [A, B],
                  dict(M=M, K=K, N=8, in_dtype=in_dtype, out_dtype=out_dtype), tag="matmul")
    info = {
        "name": "tensorcore",
        "stage_name": out.op.name,
        "loadA": (A.name, (0, 1), "row_major", in_dtype),
        "loadB": ("BPad", (0, 1), "col_major", in_dtype),
        "com": ((0, 0, 1), out_dtype),
        "store": ((0, 1), out_dtype),
        "compute_func": tcgen05_atom(in_dtype, out_dtype),
    }
    ctx.set_info(info)
    ctx.set_axis_map({
        "A.shared": ["s_0", "r_0"],
        "A.shared.wmma.matrix_a": ["s_0", "r_0"],
        "BPad.shared": ["s_1", "r_0"],
        "BPad.shared.wmma_matrix_b": ["s_1", "r_0"],
        "dense.wmma.accumulator.shared": ["s_0", "s_1"],
        "dense.wmma.accumulator": ["s_0", "s_1"],
    })
    return [out]
