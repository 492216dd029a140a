"""The DL Boost GEMM's signature and semantics (ops/x86/dense.py:6-32), run on the B200 int8 kernel."""
from ..spec import compute, placeholder, tcgen05_atom


def heron_dense(ctx, M, K, N, in_dtype, out_dtype):
    """A uint8 (M,K), B int8 (N,K), out int32; like the reference, the dtype arguments are ignored."""
    A = placeholder((M, K), name="A", dtype="uint8")
    B = placeholder((N, K), name="B", dtype="int8")
    out = compute((M, N), "int32", "dense", "gemm", [A, B],
                  dict(M=M, K=K, N=N, in_dtype="uint8", out_dtype="int32"))
    info = {
        "name": "x86_dot",
        "stage_orgination": [("dense", "addCacheWriteGlobal")],
        "com": ("dense.global", (1, 0)),
        # the reference names the VNNI 16x4 micro-kernel here; this build names its MMA atom
        "intrin": [tcgen05_atom("uint8", "int32"), 16, 4],
    }
    ctx.set_info(info)
    ctx.set_axis_map({"dense.global": ["s_0", "s_1"]})
    return [out]
