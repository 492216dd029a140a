"""The DL Boost batched GEMM (ops/x86/batch_matmul.py:6-34): uint8 x int8 -> int32."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_batch_matmul(ctx, batch, M, K, N, in_dtype, out_dtype):
    A = placeholder((batch, M, K), name="A", dtype="uint8")
    B = placeholder((batch, N, K), name="B", dtype="int8")
    out = compute((batch, M, N), "int32", "batch_matmul", "bmm", [A, B],
                  dict(batch=batch, M=M, K=K, N=N, in_dtype="uint8", out_dtype="int32"))
    info = {
        "name": "x86_dot",
        "stage_orgination": [("batch_matmul", "addCacheWriteGlobal")],
        "com": ("batch_matmul.global", (2, 1)),
        "intrin": [tcgen05_atom("uint8", "int32"), 16, 4],
    }
    ctx.set_info(info)
    ctx.set_axis_map({"batch_matmul.global": ["s_0", "s_1", "s_2"]})
    return [out]
