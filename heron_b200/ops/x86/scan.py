"""The DL Boost scan operator (ops/x86/scan.py:6-41): uint8 A against the constant int8 triangle."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_scan(ctx, M, N, K, in_dtype, out_dtype):
    """A uint8 (M,K); B int8 (N,K) constant, B[i,j] = 0 if i <= j else 1; out int32 (M,N).  Like the
    reference, the dtype arguments are ignored."""
    A = placeholder((M, K), name="A", dtype="uint8")
    out = compute((M, N), "int32", "dense", "scan", [A],
                  dict(M=M, K=K, N=N, in_dtype="uint8", out_dtype="int32"))
    info = {
        "name": "x86_dot",
        "stage_orgination": [("dense", "addCacheWriteGlobal")],
        "com": ("dense.global", (1, 0)),
        "intrin": [tcgen05_atom("uint8", "int32"), 16, 4],
    }
    ctx.set_info(info)
    ctx.set_axis_map({"dense.global": ["s_0", "s_1"]})
    return [out]
