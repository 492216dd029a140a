"""Seeded synthetic inputs for the five benchmark configurations.

The shapes are those of the reference's own experiment files (GEMM 64^3:
tests/quick_start/dlboost/quick_start.json:14; GEMM 4096^3: tests/figure6/configs/gemm.json:15;
ResNet-50 3x3 layers: tests/figure10/configs/resnet50.json:16,30; BERT score BMM:
tests/figure10/configs/bert.json:15) at the batch sizes the benchmark names.  The reference
fills its tensors with unseeded random values (tests/quick_start/dlboost/run.py:52-58); here
every tensor comes from ``numpy.random.Generator(PCG64(seed))`` with seed = 20240 + config index,
so that the oracle, the CPU baseline and the GPU kernels see identical bytes.
"""
import numpy as np

SEED_BASE = 20240

# name -> (operator registry, op name, case args, in dtype(s), out dtype)
CONFIGS = {
    "cfg1_gemm_u8s8_64": dict(index=1, platform="dlboost", op="gemm", case=[64, 64, 64],
                              in_dtype="uint8", out_dtype="int32"),
    "cfg2_gemm_f16_4096": dict(index=2, platform="tensorcore", op="gemm", case=[4096, 4096, 4096],
                               in_dtype="float16", out_dtype="float32"),
    "cfg3_conv_f16_resnet_s2": dict(index=3, platform="tensorcore", op="c2d_nhwc",
                                    case=[32, 56, 56, 64, 64, 3, 3, 1, 1, 1],
                                    in_dtype="float16", out_dtype="float16"),
    "cfg4_bmm_s8_attention": dict(index=4, platform="tensorcore", op="bmm", case=[192, 512, 64, 512],
                                  in_dtype="int8", out_dtype="int32"),
    "cfg5_conv_u8s8_resnet_s4": dict(index=5, platform="tensorcore", op="c2d_nhwc",
                                     case=[1024, 7, 7, 512, 512, 3, 3, 1, 1, 1],
                                     in_dtype="uint8", w_dtype="int8", out_dtype="int32"),
}


def rng_for(index):
    return np.random.Generator(np.random.PCG64(SEED_BASE + index))


def _ints(rng, shape, dtype):
    if np.dtype(dtype) == np.uint8:
        return rng.integers(0, 256, size=shape, dtype=np.uint8)
    return rng.integers(-128, 128, size=shape, dtype=np.int8)


def gemm_inputs(M, K, N, in_dtype, rng, b_dtype=None):
    """A (M,K), B (N,K).  fp16: A ~ N(0,1)/sqrt(K), B ~ N(0,1); integers: uniform full range."""
    if in_dtype == "float16":
        a = (rng.standard_normal((M, K), dtype=np.float32) / np.sqrt(K)).astype(np.float16)
        b = rng.standard_normal((N, K), dtype=np.float32).astype(np.float16)
    else:
        a = _ints(rng, (M, K), in_dtype)
        b = _ints(rng, (N, K), b_dtype or ("int8" if in_dtype == "uint8" else in_dtype))
    return a, b


def bmm_inputs(B, M, K, N, in_dtype, rng, b_dtype=None):
    if in_dtype == "float16":
        a = (rng.standard_normal((B, M, K), dtype=np.float32) / np.sqrt(K)).astype(np.float16)
        b = rng.standard_normal((B, N, K), dtype=np.float32).astype(np.float16)
    else:
        a = _ints(rng, (B, M, K), in_dtype)
        b = _ints(rng, (B, N, K), b_dtype or ("int8" if in_dtype == "uint8" else in_dtype))
    return a, b


def conv_inputs(N, H, W, CI, CO, KH, KW, in_dtype, rng, w_dtype=None):
    """Input NHWC, filter HWIO.  fp16: input ~ N(0,1), filter ~ N(0, 1/sqrt(KH*KW*CI))."""
    if in_dtype == "float16":
        x = rng.standard_normal((N, H, W, CI), dtype=np.float32).astype(np.float16)
        w = (rng.standard_normal((KH, KW, CI, CO), dtype=np.float32) / np.sqrt(KH * KW * CI)).astype(np.float16)
    else:
        x = _ints(rng, (N, H, W, CI), in_dtype)
        w = _ints(rng, (KH, KW, CI, CO), w_dtype or "int8")
    return x, w


def make_inputs(name, shard=None):
    """Host arrays of a named configuration; ``shard=(start, count)`` keeps only that range of
    the leading (batch / image) dimension of the activations, generated from the same stream so
    that shards of different ranks are slices of the same global tensors."""
    cfg = CONFIGS[name]
    rng = rng_for(cfg["index"])
    case = cfg["case"]
    if cfg["op"] == "gemm":
        return gemm_inputs(case[0], case[1], case[2], cfg["in_dtype"], rng)
    if cfg["op"] == "bmm":
        a, b = bmm_inputs(case[0], case[1], case[2], case[3], cfg["in_dtype"], rng)
        if shard is not None:
            s, c = shard
            a, b = a[s:s + c], b[s:s + c]
        return np.ascontiguousarray(a), np.ascontiguousarray(b)
    x, w = conv_inputs(case[0], case[1], case[2], case[3], case[4], case[5], case[6], cfg["in_dtype"],
                       rng, cfg.get("w_dtype"))
    if shard is not None:
        s, c = shard
        x = np.ascontiguousarray(x[s:s + c])
    return x, w


def work_and_bytes(name, units=None):
    """(algorithmic operations, algorithmic bytes) of one pass; ``units`` overrides the size of
    the sharded leading dimension."""
    cfg = CONFIGS[name]
    case = list(cfg["case"])
    es = 2 if cfg["in_dtype"] == "float16" else 1
    eo = {"float32": 4, "float16": 2, "int32": 4}[cfg["out_dtype"]]
    if cfg["op"] == "gemm":
        M, K, N = case
        return 2 * M * N * K, (M * K + N * K) * es + M * N * eo
    if cfg["op"] == "bmm":
        B, M, K, N = case
        if units is not None:
            B = units
        return 2 * B * M * N * K, B * ((M * K + N * K) * es + M * N * eo)
    N, H, W, CI, CO, KH, KW, s, p, d = case
    if units is not None:
        N = units
    HO = (H - ((KH - 1) * d + 1) + 2 * p) // s + 1
    WO = (W - ((KW - 1) * d + 1) + 2 * p) // s + 1
    return (2 * N * HO * WO * CO * KH * KW * CI,
            N * H * W * CI * es + KH * KW * CI * CO * es + N * HO * WO * CO * eo)
