"""The DL Boost matrix-vector product (ops/x86/gemv.py:6-33): a GEMM with one row of A."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_gemv(ctx, M, K, in_dtype, out_dtype):
    """A uint8 (1,K), B int8 (M,K), out int32 (1,M): out[0,j] = sum_k A[0,k] * B[j,k].  Like the
    reference, the dtype arguments are ignored.  It is the GEMM kernel with a single row of A."""
    A = placeholder((1, K), name="A", dtype="uint8")
    B = placeholder((M, K), name="B", dtype="int8")
    out = compute((1, M), "int32", "dense", "gemm", [A, B],
                  dict(M=1, K=K, N=M, in_dtype="uint8", out_dtype="int32"))
    info = {
        "name": "x86_dot",
        "stage_orgination": [("dense", "addCacheWriteGlobal")],
        "com": ("dense.global", (1, 0)),
        "intrin": [tcgen05_atom("uint8", "int32"), 16, 4],
    }
    ctx.set_info(info)
    ctx.set_axis_map({"dense.global": ["s_0", "s_1"]})
    return [out]
