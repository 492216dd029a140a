"""GEMM with the signature of the reference's tensor-core operator (ops/cuda/dense.py:4-54)."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_dense(ctx, M, K, N, in_dtype, out_dtype):
    """out[i,j] = sum_k A[i,k].astype(out_dtype) * B[j,k].astype(out_dtype); B is (N, K)."""
    A = placeholder((M, K), name="A", dtype=in_dtype)
    B = placeholder((N, K), name="B", dtype=in_dtype)
    out = compute((M, N), out_dtype, "dense", "gemm", [A, B],
                  dict(M=M, K=K, N=N, in_dtype=in_dtype, out_dtype=out_dtype), tag="batch_matmul")
    # Same keys as the reference hands to its scheduler (ops/cuda/dense.py:35-53); compute_func
    # names the tcgen05 atom instead of a wmma tensor expression.
    info = {
        "name": "tensorcore",
        "stage_name": out.op.name,
        "loadA": (A.name, (0, 1), "row_major", in_dtype),
        "loadB": (B.name, (0, 1), "col_major", in_dtype),
        "com": ((0, 0, 1), out_dtype),
        "store": ((0, 1), out_dtype),
        "compute_func": tcgen05_atom(in_dtype, out_dtype),
    }
    ctx.set_info(info)
    axis_map = {
        "A.shared": ["s_0", "r_0"],
        "A.shared.wmma.matrix_a": ["s_0", "r_0"],
        "B.shared": ["s_1", "r_0"],
        "B.shared.wmma_matrix_b": ["s_1", "r_0"],
        "dense.wmma.accumulator.shared": ["s_0", "s_1"],
        "dense.wmma.accumulator": ["s_0", "s_1"],
    }
    ctx.set_axis_map(axis_map)
    return [out]
