"""Batched GEMM with the reference's signature (ops/cuda/batch_matmul.py:5-56)."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_batch_matmul(ctx, batch, M, K, N, in_dtype, out_dtype):
    """out[b,i,j] = sum_k A[b,i,k] * B[b,j,k]; the reference requires batch > 1 (line 6)."""
    assert batch > 1
    A = placeholder((batch, M, K), name="A", dtype=in_dtype)
    B = placeholder((batch, N, K), name="B", dtype=in_dtype)
    out = compute((batch, M, N), out_dtype, "batch_matmul", "bmm", [A, B],
                  dict(batch=batch, M=M, K=K, N=N, in_dtype=in_dtype, out_dtype=out_dtype),
                  tag="batch_matmul")
    # The reference hard-codes 'float16' in loadA/loadB (ops/cuda/batch_matmul.py:40-41), which
    # limits its own GPU schedule to fp16; the operator math is dtype-generic and so is this one.
    info = {
        "name": "tensorcore",
        "stage_name": out.op.name,
        "loadA": (A.name, (1, 2), "row_major", in_dtype),
        "loadB": (B.name, (1, 2), "col_major", in_dtype),
        "com": ((1, 0, 2), out_dtype),
        "store": ((1, 2), out_dtype),
        "compute_func": tcgen05_atom(in_dtype, out_dtype),
    }
    ctx.set_info(info)
    axis_map = {
        "A.shared": ["s_0", "s_1", "r_0"],
        "A.shared.wmma.matrix_a": ["s_0", "s_1", "r_0"],
        "B.shared": ["s_0", "s_2", "r_0"],
        "B.shared.wmma.matrix_b": ["s_0", "s_2", "r_0"],
        "batch_matmul.wmma.accumulator.shared": ["s_0", "s_1", "s_2"],
        "batch_matmul.wmma.accumulator": ["s_0", "s_1", "s_2"],
    }
    ctx.set_axis_map(axis_map)
    return [out]
