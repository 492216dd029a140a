"""The scan operator in the reference's tensor-core form (ops/cuda/scan.py:4-59)."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_scan(ctx, M, N, K, in_dtype, out_dtype):
    """A (M,K); B (N,K) is the constant B[i,j] = 0 if i <= j else 1 (ops/cuda/scan.py:6-13), not an
    input; out[i,j] = sum_k A[i,k] * B[j,k] = sum of A[i,k] over k < j."""
    A = placeholder((M, K), name="A", dtype=in_dtype)
    out = compute((M, N), out_dtype, "dense", "scan", [A],
                  dict(M=M, K=K, N=N, in_dtype=in_dtype, out_dtype=out_dtype), tag="matmul")
    info = {
        "name": "tensorcore",
        "stage_name": out.op.name,
        "loadA": (A.name, (0, 1), "row_major", in_dtype),
        "loadB": ("B", (0, 1), "col_major", in_dtype),
        "com": ((0, 0, 1), out_dtype),
        "store": ((0, 1), out_dtype),
        "compute_func": tcgen05_atom(in_dtype, out_dtype),
    }
    ctx.set_info(info)
    ctx.set_axis_map({
        "A.shared": ["s_0", "r_0"],
        "A.shared.wmma.matrix_a": ["s_0", "r_0"],
        "B.shared": ["s_1", "r_0"],
        "B.shared.wmma_matrix_b": ["s_1", "r_0"],
        "dense.wmma.accumulator.shared": ["s_0", "s_1"],
        "dense.wmma.accumulator": ["s_0", "s_1"],
    })
    return [out]
