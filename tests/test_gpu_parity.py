"""Parity of the sm_100a kernels with the oracle, through the C ABI (ctypes), on a B200.

Bit-exact for the integer paths.  For fp16 inputs with fp32 accumulation two bounds hold at once:
every element satisfies |got - want| <= 1e-2 * |want| + atol with atol = 1e-3 * RMS(want) (the
benchmark's stated relative tolerance, with a floor so that sums that cancel to almost nothing are
not held to a relative bound), and the largest error is at most 1e-2 of the largest magnitude of
the oracle's output.  Observed errors are around 1e-6 (fp32 output) and 5e-4 (fp16 output).
"""
import os
import random

import numpy as np
import pytest
import torch

from golden_util import assert_matches, load_cases, run_case
from oracle import np_oracle as npo

pytestmark = pytest.mark.gpu

FP_TOL = 1e-2        # relative, per element and against the largest magnitude
FP_ATOL_RMS = 1e-3   # absolute floor of the per-element bound, as a fraction of RMS(want)


@pytest.fixture(scope="module")
def K(hb_lib):
    assert torch.cuda.is_available(), "GPU tests need a B200"
    from heron_b200 import kernels
    assert hb_lib.hb_sm_count() > 0, "libheron_b200.so found no sm_100 device"
    return kernels


@pytest.fixture(scope="module")
def co(oracle_libs):
    from oracle import c_oracle
    return c_oracle


@pytest.fixture(autouse=True)
def _status_clean(hb_lib):
    yield
    from heron_b200 import _lib
    assert _lib.last_status() == 0, "a bounded device-side wait ran out"


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def poison(shape, dtype):
    """Output buffers start as 0xCD bytes so that an unwritten tile cannot pass."""
    t = torch.empty(shape, dtype=dtype, device="cuda")
    t.view(torch.uint8).fill_(0xCD)
    return t


_T = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16, np.dtype(np.int32): torch.int32}


def check(got_t, want, what=""):
    got = got_t.cpu().numpy()
    assert got.shape == want.shape, what
    if want.dtype.kind in "iu":
        assert np.array_equal(got, want), "%s: %d mismatches" % (what, int((got != want).sum()))
    else:
        assert np.isfinite(got.astype(np.float32)).all(), what
        w64, diff = want.astype(np.float64), np.abs(got.astype(np.float64) - want.astype(np.float64))
        scale = max(float(np.abs(w64).max()), 1e-30)
        assert float(diff.max()) / scale <= FP_TOL, (what, float(diff.max()) / scale)
        atol = FP_ATOL_RMS * float(np.sqrt(np.mean(w64 * w64)))
        excess = diff - (FP_TOL * np.abs(w64) + atol)
        assert float(excess.max()) <= 0.0, "%s: %d elements outside |d| <= %g|want| + %g" % (
            what, int((excess > 0).sum()), FP_TOL, atol)


def k_gemm(K, a, b, out_dtype=None, knobs=None):
    od = out_dtype or (np.float32 if a.dtype == np.float16 else np.int32)
    out = poison((a.shape[0], b.shape[0]), _T[np.dtype(od)])
    K.gemm(dev(a), dev(b), out=out, knobs=knobs)
    return out


def k_bmm(K, a, b, knobs=None):
    od = torch.float32 if a.dtype == np.float16 else torch.int32
    out = poison((a.shape[0], a.shape[1], b.shape[1]), od)
    K.bmm(dev(a), dev(b), out=out, knobs=knobs)
    return out


def k_conv(K, x, w, stride, pad, dil, out_dtype=None, knobs=None):
    od = np.dtype(out_dtype or (np.float32 if x.dtype == np.float16 else np.int32))
    HO, WO = K.conv_out_hw(x.shape[1], x.shape[2], w.shape[0], w.shape[1], stride, pad, dil)
    out = poison((x.shape[0], HO, WO, w.shape[3]), _T[od])
    K.conv2d_nhwc(dev(x), dev(w), stride=stride, padding=pad, dilation=dil, out=out, knobs=knobs)
    return out


def k_conv_packed(K, x, wp, stride, pad, dil, knobs=None):
    OC, KH, KW, IC, sco, _ = wp.shape
    return K.conv2d_nhwc_packed(dev(x), dev(wp), OC * sco, KH, KW, stride=stride, padding=pad, dilation=dil,
                                sco=sco, knobs=knobs)


def rand_i8(rng, shape, signed):
    return rng.integers(-128, 128, shape).astype(np.int8) if signed else rng.integers(0, 256, shape, dtype=np.uint8)


# ---- committed golden cases ---------------------------------------------------------------
def test_golden_cases(K):
    for name, case in load_cases().items():
        got = run_case(
            name, case,
            lambda a, b: k_gemm(K, a, b), lambda a, b: k_bmm(K, a, b), lambda a, b: k_gemm(K, a, b),
            lambda x, w, s, p, d: k_conv(K, x, w, s, p, d),
            lambda x, w, s, p, d, od: k_conv(K, x, w, s, p, d, out_dtype=od),
            lambda x, w, s, p, d: k_conv_packed(K, x, w, s, p, d))
        assert_matches(name, got.cpu().numpy(), case["out"])


def test_golden_neighbour_cases(K):
    from golden_util import run_neighbour_case

    def c1d_packed(x, wp, s, p, d):
        OC, KW, IC, sco, _ = wp.shape
        return K.conv1d_nwc_packed(dev(x), dev(wp), OC * sco, KW, stride=s, padding=p, dilation=d, sco=sco)

    for name, case in load_cases("kat_neighbours.npz").items():
        got = run_neighbour_case(name, case, lambda a, x: K.gemv(dev(a), dev(x)),
                                 lambda x, w, s, p: K.conv1d_ncw(dev(x), dev(w), s, p), c1d_packed)
        assert_matches(name, got.cpu().numpy(), case["out"])


# ---- GEMM ---------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,Kd", [(64, 64, 64), (1, 16, 16), (128, 256, 128), (129, 257, 144), (300, 200, 80),
                                    (512, 512, 512), (1000, 136, 1040), (128, 36, 64)])
@pytest.mark.parametrize("a_signed,b_signed", [(False, True), (True, True), (False, False), (True, False)])
def test_gemm_int8_exact(K, co, M, N, Kd, a_signed, b_signed):
    rng = np.random.default_rng(M * 7 + N * 3 + Kd + a_signed * 2 + b_signed)
    a, b = rand_i8(rng, (M, Kd), a_signed), rand_i8(rng, (N, Kd), b_signed)
    check(k_gemm(K, a, b), co.gemm_int(a, b), "gemm int8 %s" % ((M, N, Kd),))


@pytest.mark.parametrize("M,N,Kd", [(64, 64, 64), (128, 64, 8), (130, 260, 72), (512, 384, 1024), (2048, 512, 256)])
@pytest.mark.parametrize("out_dtype", [np.float32, np.float16])
def test_gemm_fp16(K, co, M, N, Kd, out_dtype):
    rng = np.random.default_rng(M + N + Kd)
    a = (rng.standard_normal((M, Kd)) / np.sqrt(Kd)).astype(np.float16)
    b = rng.standard_normal((N, Kd)).astype(np.float16)
    check(k_gemm(K, a, b, out_dtype=out_dtype), co.gemm_f16(a, b).astype(out_dtype), "gemm f16")


@pytest.mark.parametrize("knobs", [
    dict(tile_n=32), dict(tile_n=96, stages=2), dict(tile_n=256, stages=1), dict(tile_n=128, acc_stages=1),
    dict(swizzle_bytes=64), dict(swizzle_bytes=32, tile_n=64), dict(epilogue=2), dict(epilogue=2, tile_n=160),
    dict(raster=1), dict(max_ctas=3), dict(tile_n=224, stages=3, raster=1),
    dict(cta_group=1), dict(cta_group=2), dict(cta_group=2, tile_n=64, swizzle_bytes=64), dict(cta_group=1, tile_n=256),
    dict(cta_group=2, epilogue=2, acc_stages=1), dict(cta_group=2, l2_prefetch=3), dict(cta_group=2, max_ctas=5),
    dict(epi_warps=4), dict(epi_warps=8), dict(epi_warps=8, tile_n=32), dict(epi_warps=8, tile_n=96, epilogue=2),
    dict(epi_warps=8, cta_group=2), dict(epi_warps=8, cta_group=2, tile_n=160, acc_stages=1), dict(epi_warps=8, max_ctas=2),
    dict(epi_warps=4, tile_n=256, cta_group=1), dict(epi_warps=8, tile_n=224, raster=1, epilogue=2),
])
def test_gemm_every_knob_gives_the_same_bits(K, co, knobs):
    rng = np.random.default_rng(42)
    a, b = rand_i8(rng, (640, 192), False), rand_i8(rng, (480, 192), True)
    check(k_gemm(K, a, b, knobs=knobs), co.gemm_int(a, b), str(knobs))


# ---- split-K: slices of the reduction added into a zeroed output ---------------------------
@pytest.mark.parametrize("knobs", [
    dict(split_k=2), dict(split_k=3), dict(split_k=4), dict(split_k=2, epilogue=2), dict(split_k=4, epilogue=2),
    dict(split_k=3, cta_group=1, tile_n=128), dict(split_k=2, cta_group=2, tile_n=64, swizzle_bytes=64),
    dict(split_k=4, max_ctas=6), dict(split_k=2, raster=1, max_ctas=10),
    dict(split_k=3, epi_warps=8), dict(split_k=2, epi_warps=8, epilogue=2, cta_group=2), dict(split_k=4, epi_warps=4),
])
@pytest.mark.parametrize("M,N,Kd", [(300, 200, 1040), (1024, 520, 512)])
def test_split_k_int8_exact(K, co, knobs, M, N, Kd):
    rng = np.random.default_rng(M + Kd)
    a, b = rand_i8(rng, (M, Kd), False), rand_i8(rng, (N, Kd), True)
    plan = K.plan_gemm(dev(a), dev(b), out=poison((M, N), torch.int32), knobs=knobs)
    tiles = -(-M // (128 * plan.knobs()["cta_group"])) * -(-N // plan.knobs()["tile_n"])
    units = plan.knobs()["grid"] // plan.knobs()["cta_group"]
    if tiles % max(units, 1) or tiles < units:
        assert plan.knobs()["split_k"] == knobs["split_k"]  # the path under test is the one that runs
    check(k_gemm(K, a, b, knobs=knobs), co.gemm_int(a, b), "split-K %s" % (knobs,))


def test_split_k_fp16_is_deterministic_and_close(K, co):
    rng = np.random.default_rng(77)
    M, N, Kd = 300, 264, 2048
    a = (rng.standard_normal((M, Kd)) / np.sqrt(Kd)).astype(np.float16)
    b = rng.standard_normal((N, Kd)).astype(np.float16)
    want = co.gemm_f16(a, b)
    first = None
    for _ in range(3):
        for knobs in (dict(split_k=4), dict(split_k=4, epilogue=2)):
            got = k_gemm(K, a, b, knobs=knobs)
            check(got, want, "split-K fp16")
            if first is None:
                first = got.clone()
            assert torch.equal(got, first)  # the slices of a tile add in slice order, whoever finishes first


def test_split_k_conv_and_bmm(K, co):
    rng = np.random.default_rng(5)
    x = rand_i8(rng, (6, 7, 7, 128), False)
    w = rand_i8(rng, (3, 3, 128, 128), True)
    want = co.conv2d_nhwc_int(x, w, 1, 1, 1)
    for knobs in (dict(split_k=2, conv_algo=1), dict(split_k=3, conv_algo=1, cta_group=1), dict(split_k=4, conv_algo=1, epilogue=2)):
        check(k_conv(K, x, w, 1, 1, 1, knobs=knobs), want, "conv split-K %s" % (knobs,))
    a, b = rand_i8(rng, (5, 200, 512), True), rand_i8(rng, (5, 72, 512), True)
    for knobs in (dict(split_k=2), dict(split_k=4, max_ctas=4)):
        check(k_bmm(K, a, b, knobs=knobs), co.bmm_int(a, b), "bmm split-K %s" % (knobs,))


@pytest.mark.parametrize("knobs", [
    dict(k_slices=1), dict(k_slices=2), dict(k_slices=2, cta_group=1), dict(k_slices=2, cta_group=2, stages=1),
    dict(k_slices=2, stages=2, acc_stages=1), dict(k_slices=2, split_k=2, max_ctas=6),
    dict(k_slices=2, split_k=3, cta_group=1, max_ctas=5), dict(k_slices=2, tile_n=64, swizzle_bytes=64),
    dict(k_slices=2, tile_n=128, swizzle_bytes=32, epilogue=2),
])
def test_two_k_spans_per_ring_stage(K, co, knobs):
    """One or two swizzle spans of K behind each ring barrier: K extents of 1, 3, 5 and 9 spans
    (a last stage that is half full), with split-K slices that cut the K range at odd spans."""
    rng = np.random.default_rng(sum(knobs.values()))
    for M, N, Kd in ((300, 200, 128), (300, 200, 384), (520, 328, 640), (129, 72, 1152)):
        if Kd * 8 < 128 * 8 * knobs.get("split_k", 1):
            continue  # every split-K slice keeps at least one span
        a, b = rand_i8(rng, (M, Kd), False), rand_i8(rng, (N, Kd), True)
        check(k_gemm(K, a, b, knobs=knobs), co.gemm_int(a, b), "k spans int8 %s %s" % ((M, N, Kd), knobs))
    af = (rng.standard_normal((260, 328)) / np.sqrt(328)).astype(np.float16)
    bf = rng.standard_normal((136, 328)).astype(np.float16)
    check(k_gemm(K, af, bf, knobs=knobs), co.gemm_f16(af, bf), "k spans fp16 %s" % (knobs,))
    ck = {k: v for k, v in knobs.items() if k not in ("split_k", "swizzle_bytes")}
    x, w = rand_i8(rng, (3, 9, 11, 64), False), rand_i8(rng, (3, 3, 64, 80), True)
    check(k_conv(K, x, w, (2, 1), 1, 1, knobs=dict(ck, conv_algo=1)), co.conv2d_nhwc_int(x, w, (2, 1), 1, 1),
          "k spans conv %s" % (ck,))
    a3, b3 = rand_i8(rng, (5, 200, 320), True), rand_i8(rng, (5, 72, 320), True)
    check(k_bmm(K, a3, b3, knobs=ck), co.bmm_int(a3, b3), "k spans bmm %s" % (ck,))


@pytest.mark.parametrize("knobs", [
    dict(epi_warps=8), dict(epi_warps=8, cta_group=2), dict(epi_warps=8, epilogue=2), dict(epi_warps=8, tile_n=64),
    dict(epi_warps=8, tile_n=192, acc_stages=2, max_ctas=3), dict(epi_warps=4),
])
def test_eight_epilogue_warps(K, co, knobs):
    """Two warps per 32 TMEM lanes, each draining half of a tile's 128-byte column chunks (an odd
    count leaves the first warp one more, a single chunk leaves the second none): fp16 and fp32
    outputs, ragged edges, conv through im2col loads, batched GEMM, and the library's own pick
    on a short-K shape."""
    rng = np.random.default_rng(11 + sum(knobs.values()))
    for M, N, Kd in ((300, 200, 64), (640, 488, 192), (129, 1000, 320)):
        a, b = rand_i8(rng, (M, Kd), False), rand_i8(rng, (N, Kd), True)
        check(k_gemm(K, a, b, knobs=knobs), co.gemm_int(a, b), "epi warps int8 %s %s" % ((M, N, Kd), knobs))
    af = (rng.standard_normal((260, 328)) / np.sqrt(328)).astype(np.float16)
    bf = rng.standard_normal((392, 328)).astype(np.float16)
    for od in (np.float32, np.float16):
        check(k_gemm(K, af, bf, out_dtype=od, knobs=knobs), co.gemm_f16(af, bf).astype(od), "epi warps fp16 %s" % (knobs,))
    ck = {k: v for k, v in knobs.items() if k != "tile_n"}
    x, w = rand_i8(rng, (3, 9, 11, 64), False), rand_i8(rng, (3, 3, 64, 80), True)
    check(k_conv(K, x, w, (2, 1), 1, 1, knobs=dict(ck, conv_algo=1)), co.conv2d_nhwc_int(x, w, (2, 1), 1, 1),
          "epi warps conv %s" % (ck,))
    a3, b3 = rand_i8(rng, (5, 200, 64), True), rand_i8(rng, (5, 264, 64), True)
    check(k_bmm(K, a3, b3, knobs=ck), co.bmm_int(a3, b3), "epi warps bmm %s" % (ck,))


def test_short_k_shapes_take_eight_epilogue_warps(K):
    """The library's pick: eight where a tile has fewer swizzle spans of K than column chunks."""
    a = torch.zeros((1024, 64), dtype=torch.int8, device="cuda")
    b = torch.zeros((512, 64), dtype=torch.int8, device="cuda")
    assert K.plan_gemm(a.view(torch.uint8), b, knobs=dict(tile_n=256)).knobs()["epi_warps"] == 8
    a = torch.zeros((1024, 4096), dtype=torch.int8, device="cuda")
    b = torch.zeros((512, 4096), dtype=torch.int8, device="cuda")
    assert K.plan_gemm(a.view(torch.uint8), b, knobs=dict(tile_n=256)).knobs()["epi_warps"] == 4


# ---- balanced schedule (knob balance = 2) --------------------------------------------------------
BALANCE_KNOBS = [
    dict(), dict(cta_group=1), dict(cta_group=2), dict(max_ctas=6), dict(max_ctas=10, cta_group=2),
    dict(k_slices=1, max_ctas=14), dict(k_slices=2, max_ctas=22, cta_group=1), dict(epilogue=2, max_ctas=8),
    dict(tile_n=64, max_ctas=12), dict(tile_n=128, cta_group=2, max_ctas=20, stages=2),
    dict(raster=1, max_ctas=18), dict(acc_stages=1, max_ctas=6),
    dict(epi_warps=8, max_ctas=10), dict(epi_warps=8, cta_group=2, max_ctas=14), dict(epi_warps=8, tile_n=96, epilogue=2, max_ctas=7),
    dict(epi_warps=4, max_ctas=9),
]


@pytest.mark.parametrize("knobs", BALANCE_KNOBS)
def test_balanced_schedule_gemm_and_bmm(K, co, knobs):
    """Equal runs of (tile, K stage) units per CTA pair: tiles at the ends of a run are shared with
    the neighbouring pair through partial sums left in the output.  Integer results are exact;
    fp32 results equal the oracle within tolerance and are identical from launch to launch."""
    kn = dict(knobs, balance=2)
    rng = np.random.default_rng(77 + sum(knobs.values()))
    for M, N, Kd in ((520, 328, 1152), (1000, 136, 2048), (300, 200, 640), (129, 260, 4096)):
        a, b = rand_i8(rng, (M, Kd), False), rand_i8(rng, (N, Kd), True)
        check(k_gemm(K, a, b, knobs=kn), co.gemm_int(a, b), "balanced int8 %s %s" % ((M, N, Kd), kn))
    af = (rng.standard_normal((700, 1536)) / np.sqrt(1536)).astype(np.float16)
    bf = rng.standard_normal((392, 1536)).astype(np.float16)
    first = k_gemm(K, af, bf, knobs=kn)
    check(first, co.gemm_f16(af, bf), "balanced fp16 %s" % (kn,))
    for _ in range(3):
        assert torch.equal(k_gemm(K, af, bf, knobs=kn), first), "the order of the additions is fixed"
    a3, b3 = rand_i8(rng, (7, 200, 512), True), rand_i8(rng, (7, 136, 512), True)
    check(k_bmm(K, a3, b3, knobs=kn), co.bmm_int(a3, b3), "balanced bmm %s" % (kn,))


@pytest.mark.parametrize("knobs", [dict(), dict(cta_group=1), dict(max_ctas=10), dict(k_slices=1, max_ctas=30),
                                   dict(epilogue=2, cta_group=2, max_ctas=12)])
def test_balanced_schedule_conv(K, co, knobs):
    kn = dict(knobs, balance=2, conv_algo=1)
    rng = np.random.default_rng(91 + sum(knobs.values()))
    for case in ((6, 7, 7, 128, 128, 3, 3, 1, 1, 1), (4, 14, 14, 128, 256, 3, 3, 2, 1, 1), (3, 9, 11, 64, 96, 3, 3, (2, 1), 1, 1)):
        N, H, W, CI, CO, KH, KW, st, p, d = case
        x, w = rand_i8(rng, (N, H, W, CI), False), rand_i8(rng, (KH, KW, CI, CO), True)
        check(k_conv(K, x, w, st, p, d, knobs=kn), co.conv2d_nhwc_int(x, w, st, p, d), "balanced conv %s %s" % (case, kn))
    x = rng.standard_normal((5, 10, 10, 64)).astype(np.float16)
    w = (rng.standard_normal((3, 3, 64, 64)) / 24.0).astype(np.float16)
    check(k_conv(K, x, w, 1, 1, 1, out_dtype=np.float32, knobs=kn), co.conv2d_nhwc_f16(x, w, 1, 1, 1, np.float32),
          "balanced conv fp16 %s" % (kn,))


def test_schedules_agree_on_the_sharded_shapes(K, co):
    """The per-GPU shards of the two batch-sharded benchmark configurations at 4 and 8 GPUs (256 and
    128 images; 48 and 24 batches) under the balanced schedule, against the oracle on sampled
    images / batches and through exact sum identities over every element; the library's default
    schedule and split-K forced on give the same bits."""
    from heron_b200.workloads import make_inputs
    for count in (128, 256):
        x, w = make_inputs("cfg5_conv_u8s8_resnet_s4", shard=(512, count))
        out = poison((count, 7, 7, 512), torch.int32)
        plan = K.plan_conv2d_nhwc(dev(x), dev(w), stride=1, padding=1, dilation=1, out=out, knobs=dict(balance=2))
        assert plan.knobs()["balance"] == 2, plan.knobs()
        plan.launch()
        for n in (0, 1, count // 2, count - 1):
            check(out[n:n + 1], co.conv2d_nhwc_int(x[n:n + 1], w, 1, 1, 1), "shard of %d images, image %d" % (count, n))
        got = out.cpu().numpy().astype(np.int64).sum(axis=3)
        wsum = w.astype(np.int64).sum(axis=3)
        xp = np.pad(x.astype(np.int64), ((0, 0), (1, 1), (1, 1), (0, 0)))
        want = np.zeros(got.shape, dtype=np.int64)
        for ry in range(3):
            for rx in range(3):
                want += (xp[:, ry:ry + 7, rx:rx + 7, :] * wsum[ry, rx]).sum(axis=3)
        assert np.array_equal(got, want)
        forced = k_conv(K, x, w, 1, 1, 1, knobs=dict(split_k=2, balance=1))
        assert torch.equal(forced, out), "split-K and the balanced schedule agree bit for bit"
        assert torch.equal(k_conv(K, x, w, 1, 1, 1), out), "and so does the default"
    for count in (24, 48):
        a, b = make_inputs("cfg4_bmm_s8_attention", shard=(96, count))
        out = k_bmm(K, a, b)
        for bi in (0, count // 2, count - 1):
            check(out[bi], co.gemm_int(a[bi], b[bi]), "shard of %d batches, batch %d" % (count, bi))
        got = out.cpu().numpy().astype(np.int64)
        a64, b64 = a.astype(np.int64), b.astype(np.int64)
        assert np.array_equal(got.sum(axis=2), np.einsum("bik,bk->bi", a64, b64.sum(axis=1)))
        assert np.array_equal(got.sum(axis=1), np.einsum("bjk,bk->bj", b64, a64.sum(axis=1)))
        assert torch.equal(k_bmm(K, a, b, knobs=dict(balance=2)), out)


def test_balanced_schedule_refused_for_two_byte_outputs(K):
    from heron_b200._lib import HB_ERR_KNOB, HeronB200Error
    a = torch.zeros(256, 512, dtype=torch.float16, device="cuda")
    b = torch.zeros(256, 512, dtype=torch.float16, device="cuda")
    with pytest.raises(HeronB200Error) as e:
        K.gemm(a, b, out=torch.empty(256, 256, dtype=torch.float16, device="cuda"), knobs=dict(balance=2))
    assert e.value.status == HB_ERR_KNOB


def test_split_k_rejected_where_it_cannot_add(K):
    from heron_b200._lib import HB_ERR_KNOB, HeronB200Error
    a = torch.zeros(128, 512, dtype=torch.float16, device="cuda")
    b = torch.zeros(128, 512, dtype=torch.float16, device="cuda")
    for knobs, out in ((dict(split_k=2), torch.float16), (dict(split_k=5), torch.float32),
                       (dict(split_k=2, tail_split=2), torch.float32)):
        with pytest.raises(HeronB200Error) as e:
            K.gemm(a, b, out=torch.empty(128, 128, dtype=out, device="cuda"), knobs=knobs)
        assert e.value.status == HB_ERR_KNOB


def test_gemm_rejects_bad_arguments(K):
    from heron_b200._lib import HB_ERR_KNOB, HB_ERR_SHAPE, HeronB200Error
    a, b = torch.zeros(64, 24, dtype=torch.uint8, device="cuda"), torch.zeros(64, 24, dtype=torch.int8, device="cuda")
    with pytest.raises(HeronB200Error) as e:
        K.gemm(a, b)  # K bytes not a multiple of 16
    assert e.value.status == HB_ERR_SHAPE
    a, b = torch.zeros(64, 64, dtype=torch.uint8, device="cuda"), torch.zeros(64, 64, dtype=torch.int8, device="cuda")
    with pytest.raises(HeronB200Error) as e:
        K.gemm(a, b, knobs=dict(tile_n=48))
    assert e.value.status == HB_ERR_KNOB
    with pytest.raises(HeronB200Error) as e:
        K.gemm(a, b, knobs=dict(tile_n=256, stages=12))  # more shared memory than an SM has
    assert e.value.status == HB_ERR_KNOB


# ---- batched GEMM ---------------------------------------------------------------------------
@pytest.mark.parametrize("B,M,N,Kd", [(2, 64, 64, 64), (3, 200, 96, 48), (5, 130, 40, 16), (12, 512, 512, 64)])
def test_bmm_int8_exact(K, co, B, M, N, Kd):
    rng = np.random.default_rng(B + M + N)
    a, b = rand_i8(rng, (B, M, Kd), True), rand_i8(rng, (B, N, Kd), True)
    check(k_bmm(K, a, b), co.bmm_int(a, b), "bmm")


def test_bmm_fp16(K, co):
    rng = np.random.default_rng(8)
    a = (rng.standard_normal((4, 150, 64)) / 8).astype(np.float16)
    b = rng.standard_normal((4, 72, 64)).astype(np.float16)
    check(k_bmm(K, a, b), co.bmm_f16(a, b), "bmm f16")


# ---- conv -----------------------------------------------------------------------------------
CONV_CASES = [
    # N, H, W, CI, CO, KH, KW, stride, pad, dil
    (2, 8, 8, 64, 64, 3, 3, 1, 1, 1),
    (2, 8, 8, 64, 64, 1, 1, 1, 0, 1),
    (3, 7, 7, 128, 128, 3, 3, 1, 1, 1),
    (4, 14, 14, 128, 256, 3, 3, 2, 1, 1),
    (4, 14, 14, 32, 64, 3, 3, 1, 2, 2),
    (1, 9, 11, 32, 96, 3, 3, (2, 1), 1, 1),
    (5, 5, 5, 32, 32, 5, 5, 1, 2, 1),
    (2, 12, 12, 64, 32, 3, 3, 3, 0, 1),
    (1, 3, 3, 32, 32, 3, 3, 1, 0, 1),
    (8, 56, 56, 64, 64, 3, 3, 1, 1, 1),
]


@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("cta_group", [1, 2])
def test_conv_int8_exact(K, co, case, cta_group):
    N, H, W, CI, CO, KH, KW, s, p, d = case
    rng = np.random.default_rng(hash(case[:7]) % 1000)
    x, w = rand_i8(rng, (N, H, W, CI), False), rand_i8(rng, (KH, KW, CI, CO), True)
    check(k_conv(K, x, w, s, p, d, knobs=dict(cta_group=cta_group)), co.conv2d_nhwc_int(x, w, s, p, d), str(case))


@pytest.mark.parametrize("case", CONV_CASES + [(4, 9, 9, 16, 64, 3, 3, 1, 1, 1)])
@pytest.mark.parametrize("out_dtype", [np.float32, np.float16])
def test_conv_fp16(K, co, case, out_dtype):
    N, H, W, CI, CO, KH, KW, s, p, d = case
    rng = np.random.default_rng(hash(case[:7]) % 1000 + 1)
    x = rng.standard_normal((N, H, W, CI)).astype(np.float16)
    w = (rng.standard_normal((KH, KW, CI, CO)) / np.sqrt(KH * KW * CI)).astype(np.float16)
    check(k_conv(K, x, w, s, p, d, out_dtype=out_dtype), co.conv2d_nhwc_f16(x, w, s, p, d, out_dtype), str(case))


def test_conv_s8_activations(K, co):
    rng = np.random.default_rng(77)
    x, w = rand_i8(rng, (2, 6, 6, 64), True), rand_i8(rng, (3, 3, 64, 64), True)
    check(k_conv(K, x, w, 1, 1, 1), co.conv2d_nhwc_int(x, w, 1, 1, 1), "s8 x s8 conv")


@pytest.mark.parametrize("sco,fmt", [(64, "OhwI64o4i"), (48, "OhwI48o4i"), (32, "OhwI32o4i")])
def test_conv_packed_x86_format(K, co, sco, fmt):
    rng = np.random.default_rng(sco)
    x = rand_i8(rng, (3, 7, 7, 64), False)
    w = rand_i8(rng, (3, 3, 64, 192), True)
    wp = npo.pack_filter_x86(w, sco)
    got = k_conv_packed(K, x, wp, 1, 1, 1)
    assert tuple(got.shape) == (3, 7, 7, 192 // sco, sco)
    check(got, co.conv2d_nhwc_packed(x, wp, 1, 1, 1), fmt)


def test_conv_rejects_unsupported_channels(K):
    from heron_b200._lib import HB_ERR_SHAPE, HeronB200Error
    x = torch.zeros(1, 5, 5, 16, dtype=torch.uint8, device="cuda")  # 16 bytes of channels
    w = torch.zeros(3, 3, 16, 16, dtype=torch.int8, device="cuda")
    with pytest.raises(HeronB200Error) as e:
        K.conv2d_nhwc(x, w, 1, 1, 1)
    assert e.value.status == HB_ERR_SHAPE


# ---- through the reference-facing interface ----------------------------------------------------
def _task(registry, op, args, codegen):
    from heron_b200.config import Config
    from heron_b200.task import Task
    t = Task("T", registry.getOpFromName(op), args, "cuda")
    cfg = Config()
    cfg.codegen_type = codegen
    cfg.log_dir = None
    t.config = cfg
    t.make_stage_schedules()
    return t


def test_task_random_knob_points_agree(K, co):
    """Eight random feasible points of the knob space all produce the oracle's bits."""
    from heron_b200.ops import cuda as heron_cuda
    t = _task(heron_cuda, "bmm", [6, 384, 64, 320, "int8", "int32"], "GPU_TENSOR_CORE")
    rng = np.random.default_rng(21)
    a, b = rand_i8(rng, (6, 384, 64), True), rand_i8(rng, (6, 320, 64), True)
    want = co.bmm_int(a, b)
    random.seed(21)
    ta, tb = dev(a), dev(b)
    for _ in range(8):
        t.knob_manager.randSample()
        handle, args = t.instantiate(t.knob_manager)
        out = poison(args[-1].shape, torch.int32)
        handle(ta, tb, out)
        check(out, want, str(handle.knobs))


@pytest.mark.parametrize("case", [(16, 28, 28, 128, 128, 3, 3, 1, 1, 2), (16, 14, 14, 256, 512, 1, 1, 2, 0, 2),
                                  (16, 20, 20, 64, 64, 3, 3, 1, 2, 2), (8, 17, 17, 32, 64, 3, 3, 2, 3, 3)])
def test_dilated_conv_through_both_registries(K, co, case):
    """The "dil" operator (the reference's dilated-conv benchmark cases, shapes shortened): the
    tensor-core form in fp16 and the DL Boost form with the packed int8 filter."""
    from heron_b200.ops import cuda as heron_cuda, x86 as heron_cpu
    N, H, W, CI, CO, KH, KW, s, p, d = case
    rng = np.random.default_rng(sum(case))
    t = _task(heron_cuda, "dil", list(case) + ["float16", "float16"], "GPU_TENSOR_CORE")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    x = rng.standard_normal((N, H, W, CI)).astype(np.float16)
    w = (rng.standard_normal((KH, KW, CI, CO)) / np.sqrt(KH * KW * CI)).astype(np.float16)
    out = poison(args[-1].shape, torch.float16)
    handle(dev(x), dev(w), out)
    check(out, co.conv2d_nhwc_f16(x, w, s, p, d, out_dtype=np.float16), "dil fp16 %s" % (case,))
    if CO % 64 == 0 and CI % 4 == 0:
        t = _task(heron_cpu, "dil", list(case) + ["OhwI64o4i", "uint8", "int32"], "CPU")
        t.knob_manager.randSample()
        handle, args = t.instantiate(t.knob_manager)
        xi, wi = rand_i8(rng, (N, H, W, CI), False), rand_i8(rng, (KH, KW, CI, CO), True)
        wp = npo.pack_filter_x86(wi, 64)
        out = poison(args[-1].shape, torch.int32)
        handle(dev(xi), dev(wp), out)
        check(out, co.conv2d_nhwc_packed(xi, wp, s, p, d), "dil x86 %s" % (case,))


# ---- gemv and the 1-D convolutions: operators next to the hot path on the same kernels --------
@pytest.mark.parametrize("M,Kd", [(512, 16), (1024, 256), (256, 1024), (130, 80)])
def test_gemv_both_forms(K, co, M, Kd):
    """The reference's gemv cases (plus a ragged one): tensor-core form (M,8) in fp16 and int8, and
    the DL Boost form (1,M) through its registry."""
    from heron_b200.ops import cuda as heron_cuda, x86 as heron_cpu
    rng = np.random.default_rng(M + Kd)
    a = (rng.standard_normal((M, Kd)) / np.sqrt(Kd)).astype(np.float16)
    x = rng.standard_normal((1, Kd)).astype(np.float16)
    for od in (np.float32, np.float16):
        t = _task(heron_cuda, "gemv", [M, Kd, "float16", np.dtype(od).name], "GPU_TENSOR_CORE")
        t.knob_manager.randSample()
        handle, args = t.instantiate(t.knob_manager)
        out = poison((M, 8), _T[np.dtype(od)])
        handle(dev(a), dev(x), out)
        check(out, co.gemv(a, x, od), "gemv fp16 -> %s %s" % (np.dtype(od).name, handle.knobs))
        assert not out[:, 1:].any()
    ai, xi = rand_i8(rng, (M, Kd), False), rand_i8(rng, (1, Kd), True)
    out = poison((M, 8), torch.int32)
    K.gemv(dev(ai), dev(xi), out=out)
    check(out, co.gemv(ai, xi), "gemv int8")
    plan = K.plan_gemv(dev(ai), dev(xi), out=poison((M, 8), torch.int32))
    check(plan.launch(), co.gemv(ai, xi), "gemv int8 plan")
    t = _task(heron_cpu, "gemv", [M, Kd, "uint8", "int32"], "CPU")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    a1, b1 = rand_i8(rng, (1, Kd), False), rand_i8(rng, (M, Kd), True)
    out = poison((1, M), torch.int32)
    handle(dev(a1), dev(b1), out)
    check(out, co.gemm_int(a1, b1), "x86 gemv")


@pytest.mark.parametrize("M,N,Kd", [(16, 512, 128), (1024, 16, 256), (256, 1024, 256), (512, 256, 16), (100, 72, 48)])
def test_scan_both_forms(K, co, M, N, Kd):
    """The reference's scan cases (S5 shortened to a ragged one): the constant triangular operand is
    written by a kernel of the plan, then the GEMM kernel runs."""
    from heron_b200.ops import cuda as heron_cuda, x86 as heron_cpu
    rng = np.random.default_rng(M + N + Kd)
    a = (rng.standard_normal((M, Kd)) / np.sqrt(Kd)).astype(np.float16)
    for od in (np.float32, np.float16):
        t = _task(heron_cuda, "scan", [M, N, Kd, "float16", np.dtype(od).name], "GPU_TENSOR_CORE")
        t.knob_manager.randSample()
        handle, args = t.instantiate(t.knob_manager)
        assert [tuple(x.shape) for x in args] == [(M, Kd), (M, N)]
        out = poison((M, N), _T[np.dtype(od)])
        handle(dev(a), out)
        check(out, co.scan(a, N, od), "scan fp16 -> %s %s" % (np.dtype(od).name, handle.knobs))
    t = _task(heron_cpu, "scan", [M, N, Kd, "int8", "int32"], "CPU")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    ai = rand_i8(rng, (M, Kd), False)
    out = poison((M, N), torch.int32)
    plan = handle.plan(dev(ai), out)
    check(plan.launch(), co.scan(ai, N), "x86 scan %s" % (handle.knobs,))


@pytest.mark.parametrize("case", [(16, 892, 64, 128, 3, 1, 4), (4, 100, 512, 512, 3, 1, 32), (8, 77, 48, 64, 1, 1, 0),
                                  (2, 200, 3, 32, 7, 2, 3), (16, 223, 128, 256, 1, 2, 0)])
def test_conv1d_ncw(K, co, case):
    """(N, W, CI, CO, KW, stride, pad): the reference's c1d cases shortened, a 3-channel input and
    strided ones; padding wider than the filter is part of the reference's own cases."""
    from heron_b200.ops import cuda as heron_cuda
    N, W, CI, CO, KW, s, p = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, CI, W)).astype(np.float16)
    w = (rng.standard_normal((CO, CI, KW)) / np.sqrt(CI * KW)).astype(np.float16)
    if CI % 16 == 0:
        t = _task(heron_cuda, "c1d", [N, W, CI, CO, KW, s, p, 1, "float16", "float16"], "GPU_TENSOR_CORE")
        t.knob_manager.randSample()
        handle, args = t.instantiate(t.knob_manager)
        out = poison(args[-1].shape, torch.float16)
        handle(dev(x), dev(w), out)
        check(out, co.conv1d_ncw(x, w, s, p, np.float16), "c1d fp16 %s %s" % (case, handle.knobs))
    check(K.conv1d_ncw(dev(x), dev(w), s, p), co.conv1d_ncw(x, w, s, p), "c1d fp32 out %s" % (case,))
    xi, wi = rand_i8(rng, (N, CI, W), False), rand_i8(rng, (CO, CI, KW), True)
    plan = K.plan_conv1d_ncw(dev(xi), dev(wi), s, p)
    check(plan.launch(), co.conv1d_ncw(xi, wi, s, p), "c1d int8 %s" % (case,))


@pytest.mark.parametrize("case", [(1, 892, 512, 1024, 1, 1, 0, 1, 64), (1, 892, 512, 512, 3, 1, 4, 2, 64),
                                  (2, 300, 96, 64, 3, 1, 16, 8, 48), (3, 57, 32, 64, 5, 2, 3, 1, 32)])
def test_conv1d_nwc_packed_through_the_x86_registry(K, co, case):
    """(batch, W, co, ci, kernel, stride, pad, dilation, sco) in the reference's argument order."""
    from heron_b200.ops import x86 as heron_cpu
    N, W, CO, CI, KW, s, p, d, sco = case
    rng = np.random.default_rng(sum(case))
    x = rand_i8(rng, (N, W, CI), False)
    w = rand_i8(rng, (KW, CI, CO), True)
    wp = npo.pack_filter_x86_1d(w, sco)
    t = _task(heron_cpu, "c1d", [N, W, CO, CI, KW, s, p, d, "OwI%do4i" % sco, "uint8", "int32"], "CPU")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    assert tuple(args[1].shape) == wp.shape
    out = poison(args[-1].shape, torch.int32)
    handle(dev(x), dev(wp), out)
    check(out, co.conv1d_nwc_packed(x, wp, s, p, d), "x86 c1d %s %s" % (case, handle.knobs))


def test_quick_start_config_through_x86_interface(K, co):
    """Configuration 1: the DL Boost quick-start GEMM (64^3, uint8 x int8 -> int32)."""
    from heron_b200.ops import x86 as heron_cpu
    from heron_b200.workloads import make_inputs
    t = _task(heron_cpu, "gemm", [64, 64, 64, "int8", "int32"], "CPU")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    a, b = make_inputs("cfg1_gemm_u8s8_64")
    assert (a.dtype, b.dtype) == (np.uint8, np.int8)
    out = poison(args[-1].shape, torch.int32)
    plan = handle.plan(dev(a), dev(b), out)
    plan.launch()
    first = out.clone()
    out.view(torch.uint8).fill_(0xCD)
    plan.launch()
    assert torch.equal(first, out), "relaunching a plan changed the result"
    check(out, co.gemm_int(a, b), "cfg1")


def test_small_immediate_calls_reuse_their_plan(K, co):
    """A built operator called again on the same small buffers launches the plan of the first call
    (no tensor maps re-encoded); new contents in those buffers give new results, other buffers
    get a plan of their own."""
    from heron_b200.ops import x86 as heron_cpu
    t = _task(heron_cpu, "gemm", [64, 64, 64, "uint8", "int32"], "CPU")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    rng = np.random.default_rng(64)
    a, b = rand_i8(rng, (64, 64), False), rand_i8(rng, (64, 64), True)
    ta, tb, out = dev(a), dev(b), poison((64, 64), torch.int32)
    handle(ta, tb, out)
    check(out, co.gemm_int(a, b), "first call")
    assert len(handle._small_plans) == 1
    a2 = rand_i8(rng, (64, 64), False)
    ta.copy_(torch.from_numpy(a2))
    handle(ta, tb, out)
    check(out, co.gemm_int(a2, b), "second call, same buffers")
    assert len(handle._small_plans) == 1
    out2 = poison((64, 64), torch.int32)
    handle(ta, tb, out2)
    check(out2, co.gemm_int(a2, b), "other output buffer")
    assert len(handle._small_plans) == 2


# ---- the benchmark configurations at full size -----------------------------------------------
def test_cfg2_gemm_fp16_4096_full_size(K, co):
    """Full 4096^3: 48 sampled rows against the oracle, every element through a row-sum identity
    sum_j C[i,j] = sum_k A[i,k] * (sum_j B[j,k]) evaluated in float64."""
    from heron_b200.workloads import make_inputs
    a, b = make_inputs("cfg2_gemm_f16_4096")
    out = k_gemm(K, a, b)
    rows = np.random.default_rng(2).choice(4096, 48, replace=False)
    want = co.gemm_f16(a[rows], b)
    check(out[torch.from_numpy(rows).cuda()], want, "cfg2 sampled rows")
    got = out.cpu().numpy().astype(np.float64)
    colsum_b = b.astype(np.float64).sum(axis=0)
    want_rowsum = a.astype(np.float64) @ colsum_b
    assert np.abs(got.sum(axis=1) - want_rowsum).max() <= 1e-3 * np.abs(b.astype(np.float64)).sum() / 4096 * 64
    rowsum_a = a.astype(np.float64).sum(axis=0)
    want_colsum = b.astype(np.float64) @ rowsum_a
    assert np.abs(got.sum(axis=0) - want_colsum).max() <= 1e-2 * max(1.0, np.abs(want_colsum).max())


def test_cfg4_bmm_int8_full_size(K, co):
    """Full 192 x 512 x 64 x 512: four whole batches bit-exact against the oracle, every element
    through exact integer row- and column-sum identities."""
    from heron_b200.workloads import make_inputs
    a, b = make_inputs("cfg4_bmm_s8_attention")
    out = k_bmm(K, a, b)
    for bi in (0, 77, 130, 191):
        check(out[bi], co.gemm_int(a[bi], b[bi]), "cfg4 batch %d" % bi)
    got = out.cpu().numpy().astype(np.int64)
    a64, b64 = a.astype(np.int64), b.astype(np.int64)
    assert np.array_equal(got.sum(axis=2), np.einsum("bik,bk->bi", a64, b64.sum(axis=1)))
    assert np.array_equal(got.sum(axis=1), np.einsum("bjk,bk->bj", b64, a64.sum(axis=1)))


def test_cfg3_conv_fp16_full_size(K, co):
    from heron_b200.workloads import make_inputs
    x, w = make_inputs("cfg3_conv_f16_resnet_s2")
    out = k_conv(K, x, w, 1, 1, 1, out_dtype=np.float16)
    for n in (0, 13, 31):
        check(out[n:n + 1], co.conv2d_nhwc_f16(x[n:n + 1], w, 1, 1, 1, np.float16), "cfg3 image %d" % n)
    # channel-sum identity over every output element, in float64 against the fp16-rounded result
    got = out.cpu().numpy().astype(np.float64).sum(axis=3)
    wsum = w.astype(np.float64).sum(axis=3, keepdims=True)
    xp = np.pad(x.astype(np.float64), ((0, 0), (1, 1), (1, 1), (0, 0)))
    want = np.zeros(got.shape)
    for ry in range(3):
        for rx in range(3):
            want += (xp[:, ry:ry + 56, rx:rx + 56, :] * wsum[ry, rx, :, 0]).sum(axis=3)
    assert np.abs(got - want).max() <= 64 * 2e-3 * np.abs(out.cpu().numpy().astype(np.float64)).max()


def test_cfg5_conv_int8_full_size(K, co):
    """Full N=1024: six whole images bit-exact against the oracle, every element through the
    exact channel-sum identity sum_f out[n,y,x,f] = conv(in, sum_f w)."""
    from heron_b200.workloads import make_inputs
    x, w = make_inputs("cfg5_conv_u8s8_resnet_s4")
    out = k_conv(K, x, w, 1, 1, 1)
    for n in (0, 1, 511, 512, 1000, 1023):
        check(out[n:n + 1], co.conv2d_nhwc_int(x[n:n + 1], w, 1, 1, 1), "cfg5 image %d" % n)
    got = out.cpu().numpy().astype(np.int64).sum(axis=3)
    wsum = w.astype(np.int64).sum(axis=3)  # (3,3,512)
    xp = np.pad(x.astype(np.int64), ((0, 0), (1, 1), (1, 1), (0, 0)))
    want = np.zeros(got.shape, dtype=np.int64)
    for ry in range(3):
        for rx in range(3):
            want += (xp[:, ry:ry + 7, rx:rx + 7, :] * wsum[ry, rx]).sum(axis=3)
    assert np.array_equal(got, want)


def test_cfg5_through_the_x86_operator(K, co):
    """The same layer through the DL Boost operator's interface: packed filter, 5-D output."""
    from heron_b200.ops import x86 as heron_cpu
    from heron_b200.workloads import conv_inputs, rng_for
    t = _task(heron_cpu, "c2d", [16, 7, 7, 512, 512, 3, 3, 1, 1, 1, "OhwI64o4i", "uint8", "int32"], "CPU")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    x, w = conv_inputs(16, 7, 7, 512, 512, 3, 3, "uint8", rng_for(5))
    wp = npo.pack_filter_x86(w, 64)
    assert tuple(args[1].shape) == wp.shape
    out = poison(args[-1].shape, torch.int32)
    handle(dev(x), dev(wp), out)
    check(out, co.conv2d_nhwc_packed(x, wp, 1, 1, 1), "x86 c2d")


def test_tuning_run_on_device_with_the_verify_hook(K, co, tmp_path):
    """A short CGA run measured with CUDA events, every candidate checked against the oracle
    through the reference's verify hook (Task.set_verify_func), then the best record re-applied."""
    import json
    import os
    from heron_b200.config import Config
    from heron_b200.environment import Env
    from heron_b200.ops import cuda as heron_cuda
    from heron_b200.runner import LocalRunner, measure_option
    cfg = Config()
    cfg.out_name, cfg.opt_method, cfg.max_trials = str(tmp_path), "CGA", 12
    cfg.measure_time_per_round, cfg.pop_num, cfg.select_num, cfg.iter_walks, cfg.parallel = 6, 24, 12, 2, False
    cfg.codegen_type = "GPU_TENSOR_CORE"
    env = Env(measure_option(runner=LocalRunner(number=5, repeat=3)), cfg)
    task = env.createTask("B", heron_cuda.getOpFromName("bmm"), [4, 256, 64, 256, "int8", "int32"], "cuda")

    def reference(args):
        rng = np.random.default_rng(5)
        a, b = rand_i8(rng, (4, 256, 64), True), rand_i8(rng, (4, 256, 64), True)
        return [a, b], co.bmm_int(a, b)

    task.set_verify_func(reference, rtol=0.0)
    random.seed(5)
    np.random.seed(5)
    env.tune("B")
    rows = [json.loads(r) for r in open(os.path.join(cfg.log_dir, "records.txt"))]
    assert len(rows) >= 6 and all(r["perf"] > 0 for r in rows), "a candidate failed or gave a wrong result"
    handle, args = task.apply_best(os.path.join(cfg.log_dir, "records.txt"))
    a, b = task.ref_input
    out = poison(args[-1].shape, torch.int32)
    handle(dev(a), dev(b), out)
    check(out, task.ref_output, "best record")


@pytest.mark.parametrize("op,args", [
    ("bmm", [4, 256, 64, 256, "int8", "int32"]),
    ("gemm", [640, 192, 480, "int8", "int32"]),
    ("c2d_nhwc", [8, 9, 9, 64, 128, 3, 3, 1, 1, 1, "int8", "int32"]),
])
def test_many_random_knob_points(K, co, op, args):
    """Sixty distinct feasible points of each operator's knob space, all bit-exact.  (A sweep like
    this found a misaligned epilogue staging buffer for CTA pairs with 32-byte swizzle.)"""
    from heron_b200.ops import cuda as heron_cuda
    t = _task(heron_cuda, op, args, "GPU_TENSOR_CORE")
    rng = np.random.default_rng(len(args))
    if op == "bmm":
        ins = [rand_i8(rng, (4, 256, 64), True), rand_i8(rng, (4, 256, 64), True)]
        want = co.bmm_int(*ins)
    elif op == "gemm":
        ins = [rand_i8(rng, (640, 192), True), rand_i8(rng, (480, 192), True)]
        want = co.gemm_int(*ins)
    else:
        ins = [rand_i8(rng, (8, 9, 9, 64), True), rand_i8(rng, (3, 3, 64, 128), True)]
        want = co.conv2d_nhwc_int(ins[0], ins[1], 1, 1, 1)
    tin = [dev(i) for i in ins]
    random.seed(17)
    seen = set()
    for _ in range(200):
        if len(seen) >= 60:
            break
        t.knob_manager.randSample()
        handle, targs = t.instantiate(t.knob_manager)
        key = tuple(sorted(handle.knobs.items()))
        if key in seen:
            continue
        seen.add(key)
        out = poison(targs[-1].shape, torch.int32)
        handle(*tin, out)
        check(out, want, str(handle.knobs))
    assert len(seen) >= 40


@pytest.mark.parametrize("op,args", [
    ("gemm", [300, 328, 264, "float16", "float32"]),
    ("bmm", [16, 64, 64, 320, "float16", "float16"]),
    ("c2d_nhwc", [16, 14, 14, 64, 128, 3, 3, 1, 1, 1, "float16", "float16"]),
    ("c2d_nhwc", [16, 9, 9, 64, 96, 3, 3, 2, 1, 1, "float16", "float32"]),
])
def test_many_random_knob_points_fp16(K, co, op, args):
    """Forty distinct feasible points of the knob space per operator, fp16 operands with fp16 and
    fp32 outputs: every point the constraint model calls feasible runs and stays within the bounds."""
    from heron_b200.ops import cuda as heron_cuda
    t = _task(heron_cuda, op, args, "GPU_TENSOR_CORE")
    rng = np.random.default_rng(len(args) + args[1])
    od = np.float16 if args[-1] == "float16" else np.float32
    if op == "gemm":
        M, Kd, N = args[:3]
        ins = [(rng.standard_normal((M, Kd)) / np.sqrt(Kd)).astype(np.float16), rng.standard_normal((N, Kd)).astype(np.float16)]
        want = co.gemm_f16(*ins).astype(od)
    elif op == "bmm":
        B, M, Kd, N = args[:4]
        ins = [(rng.standard_normal((B, M, Kd)) / np.sqrt(Kd)).astype(np.float16),
               rng.standard_normal((B, N, Kd)).astype(np.float16)]
        want = co.bmm_f16(*ins).astype(od)
    else:
        N, H, W, CI, CO, KH, KW, s, p, d = args[:10]
        ins = [rng.standard_normal((N, H, W, CI)).astype(np.float16),
               (rng.standard_normal((KH, KW, CI, CO)) / np.sqrt(KH * KW * CI)).astype(np.float16)]
        want = co.conv2d_nhwc_f16(ins[0], ins[1], s, p, d, od)
    tin = [dev(i) for i in ins]
    random.seed(29)
    seen = set()
    for _ in range(160):
        if len(seen) >= 40:
            break
        t.knob_manager.randSample()
        handle, targs = t.instantiate(t.knob_manager)
        key = tuple(sorted(handle.knobs.items()))
        if key in seen:
            continue
        seen.add(key)
        out = poison(targs[-1].shape, torch.float16 if od == np.float16 else torch.float32)
        handle(*tin, out)
        check(out, want, str(handle.knobs))
    assert len(seen) >= 25


STRIP_CASES = [
    # N, H, W, CI, CO, KH, KW, pad, dil  (stride 1; filter + two strips fit shared memory)
    (2, 8, 8, 64, 64, 3, 3, 1, 1),
    (8, 56, 56, 64, 64, 3, 3, 1, 1),
    (2, 12, 12, 64, 64, 3, 3, 0, 1),
    (1, 100, 100, 64, 64, 1, 1, 0, 1),
    (3, 13, 9, 64, 128, 3, 3, 2, 2),
    (2, 57, 31, 128, 64, 3, 1, 1, 1),
    (2, 126, 5, 64, 64, 3, 3, 1, 1),
]


@pytest.mark.parametrize("case", STRIP_CASES)
def test_conv_strip_algorithm_fp16(K, co, case):
    """The resident-filter / halo-strip conv kernel (conv_algo 2) against the oracle, and against
    the implicit-GEMM kernel (conv_algo 1) on the same inputs."""
    N, H, W, CI, CO, KH, KW, p, d = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, H, W, CI)).astype(np.float16)
    w = (rng.standard_normal((KH, KW, CI, CO)) / np.sqrt(KH * KW * CI)).astype(np.float16)
    for od in (np.float32, np.float16):
        want = co.conv2d_nhwc_f16(x, w, 1, p, d, od)
        check(k_conv(K, x, w, 1, p, d, out_dtype=od, knobs=dict(conv_algo=2)), want, "strip %s" % (case,))
        check(k_conv(K, x, w, 1, p, d, out_dtype=od, knobs=dict(conv_algo=1)), want, "im2col %s" % (case,))


@pytest.mark.parametrize("case", [(3, 7, 7, 128, 128, 3, 3, 1, 1), (4, 28, 28, 128, 128, 3, 3, 1, 1),
                                  (2, 30, 30, 256, 128, 1, 1, 0, 1)])
def test_conv_strip_algorithm_int8(K, co, case):
    N, H, W, CI, CO, KH, KW, p, d = case
    rng = np.random.default_rng(sum(case))
    x, w = rand_i8(rng, (N, H, W, CI), False), rand_i8(rng, (KH, KW, CI, CO), True)
    check(k_conv(K, x, w, 1, p, d, knobs=dict(conv_algo=2)), co.conv2d_nhwc_int(x, w, 1, p, d), "strip int8")


def test_conv_strip_walks_its_whole_ring(K, co):
    """One CTA takes every tile in turn, so each barrier of a deep strip ring is used and reused
    (14x14 images leave room for five strip buffers beside the filter and the staging tile)."""
    rng = np.random.default_rng(1414)
    x = rng.standard_normal((8, 14, 14, 64)).astype(np.float16)
    w = (rng.standard_normal((3, 3, 64, 64)) / 24.0).astype(np.float16)
    out = poison((8, 14, 14, 64), torch.float32)
    plan = K.plan_conv2d_nhwc(dev(x), dev(w), stride=1, padding=1, dilation=1, out=out,
                              knobs=dict(conv_algo=2, max_ctas=1))
    kn = plan.knobs()
    assert kn["conv_algo"] == 2 and kn["stages"] >= 5 and kn["grid"] == 1, kn
    plan.launch()
    check(out, co.conv2d_nhwc_f16(x, w, 1, 1, 1, np.float32), "strip ring walk")


def test_conv_strip_refused_when_it_does_not_apply(K):
    from heron_b200._lib import HB_ERR_KNOB, HeronB200Error
    x = torch.zeros(2, 14, 14, 128, dtype=torch.float16, device="cuda")
    w = torch.zeros(3, 3, 128, 256, dtype=torch.float16, device="cuda")  # 576 KiB filter
    with pytest.raises(HeronB200Error) as e:
        K.conv2d_nhwc(x, w, 1, 1, 1, knobs=dict(conv_algo=2))
    assert e.value.status == HB_ERR_KNOB
    w = torch.zeros(3, 3, 128, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(HeronB200Error) as e:
        K.conv2d_nhwc(x, w, 2, 1, 1, knobs=dict(conv_algo=2))  # stride 2
    assert e.value.status == HB_ERR_KNOB
    K.conv2d_nhwc(x, w, 2, 1, 1)  # the default falls back to the implicit-GEMM kernel


def test_default_picks_a_strip_kernel_for_resnet_stage2(K):
    x = torch.zeros(8, 56, 56, 64, dtype=torch.float16, device="cuda")
    w = torch.zeros(3, 3, 64, 64, dtype=torch.float16, device="cuda")
    assert K.plan_conv2d_nhwc(x, w, 1, 1, 1).knobs()["conv_algo"] == 4   # fp16, 64 channels out, 3x3: filter rows fused
    assert K.plan_conv2d_nhwc(x, w, 1, 1, 1, out_dtype=torch.float32).knobs()["conv_algo"] == 4
    xw = torch.zeros(2, 112, 112, 64, dtype=torch.float16, device="cuda")
    assert K.plan_conv2d_nhwc(xw, w, 1, 1, 1, out_dtype=torch.float16).knobs()["conv_algo"] == 4
    # (one image row per tile and a 4-byte output: the plain strip kernel)
    assert K.plan_conv2d_nhwc(xw, w, 1, 1, 1, out_dtype=torch.float32).knobs()["conv_algo"] == 2
    w22 = torch.zeros(2, 2, 64, 64, dtype=torch.float16, device="cuda")
    assert K.plan_conv2d_nhwc(x, w22, 1, 1, 1, out_dtype=torch.float16).knobs()["conv_algo"] == 3  # not a three-tap row: the wide one
    x80 = torch.zeros(2, 80, 80, 64, dtype=torch.float16, device="cuda")
    assert K.plan_conv2d_nhwc(x80, w, 1, 1, 1, out_dtype=torch.float16).knobs()["conv_algo"] == 3  # 64 % of the MMA rows: the wide one
    assert K.plan_conv2d_nhwc(x80, w, 1, 1, 1, out_dtype=torch.float32).knobs()["conv_algo"] == 4
    w128 = torch.zeros(3, 3, 64, 128, dtype=torch.float16, device="cuda")
    x28 = torch.zeros(4, 28, 28, 64, dtype=torch.float16, device="cuda")
    assert K.plan_conv2d_nhwc(x28, w128, 1, 1, 1, out_dtype=torch.float16).knobs()["conv_algo"] == 3  # 128 channels out: the wide one
    xi = torch.zeros(4, 28, 28, 128, dtype=torch.uint8, device="cuda")
    wi = torch.zeros(3, 3, 128, 128, dtype=torch.int8, device="cuda")
    assert K.plan_conv2d_nhwc(xi, wi, 1, 1, 1).knobs()["conv_algo"] == 2  # integer operands: pixels on M
    x = torch.zeros(16, 7, 7, 512, dtype=torch.uint8, device="cuda")
    w = torch.zeros(3, 3, 512, 512, dtype=torch.int8, device="cuda")
    assert K.plan_conv2d_nhwc(x, w, 1, 1, 1).knobs()["conv_algo"] == 1


NCHW_CASES = [
    # N, CI, H, W, CO, KH, KW, stride, pad
    (2, 3, 32, 32, 64, 7, 7, 2, 3),      # the first-layer shape family (3 input channels)
    (2, 64, 14, 14, 64, 3, 3, 1, 1),
    (2, 64, 14, 14, 256, 1, 1, 1, 0),
    (2, 256, 14, 14, 128, 1, 1, 2, 0),
    (3, 16, 9, 11, 40, 3, 3, (2, 1), 1),
    (2, 32, 9, 13, 48, 1, 1, (2, 3), 0),   # strided 1x1: the glue keeps only the pixels the conv reads
    (1, 64, 28, 28, 32, 1, 1, 2, 0),
    # few input channels: the form where a whole filter row is one K block
    (2, 3, 30, 41, 32, 3, 3, 1, 1),
    (1, 1, 20, 20, 16, 5, 5, (1, 2), 2),
    (2, 4, 18, 18, 64, 3, 8, (2, 3), 0),
    (2, 8, 12, 23, 24, 2, 2, 1, 1),
    (3, 3, 16, 9, 64, 7, 7, 2, 3),        # narrower than the filter is wide plus padding
    # 1x1, stride 1, 16-byte image rows: a batched GEMM on the NCHW tensors as they are, no layout pass
    (2, 64, 16, 16, 256, 1, 1, 1, 0),
    (3, 128, 12, 20, 72, 1, 1, 1, 0),
    (2, 72, 28, 28, 40, 1, 1, 1, 0),
    (5, 512, 8, 12, 320, 1, 1, 1, 0),
    (1, 1024, 56, 56, 64, 1, 1, 1, 0),
]


@pytest.mark.parametrize("case", NCHW_CASES)
def test_conv_nchw_fp16(K, co, case):
    N, CI, H, W, CO, KH, KW, s, p = case
    rng = np.random.default_rng(sum(x if isinstance(x, int) else 3 for x in case))
    x = rng.standard_normal((N, CI, H, W)).astype(np.float16)
    w = (rng.standard_normal((CO, CI, KH, KW)) / np.sqrt(CI * KH * KW)).astype(np.float16)
    for od, tdt in ((np.float32, torch.float32), (np.float16, torch.float16)):
        want = co.conv2d_nchw(x, w, s, p, od)
        out = poison(want.shape, tdt)
        K.conv2d_nchw(dev(x), dev(w), stride=s, padding=p, out=out)
        check(out, want, "nchw %s" % (case,))


# Layers of the other two published networks (VGG-16, Inception-v3; the table files under
# heron_b200/configs/), at a batch the oracle finishes in seconds: odd image sizes (299, 149, 73,
# 35, 17), 1x7 and 7x1 windows with the operator's single padding number applied to both axes,
# channel counts that are not powers of two, stride 2 without padding.
NETWORK_LAYER_CASES = [
    (1, 3, 299, 299, 32, 3, 3, 2, 0),
    (1, 32, 149, 149, 32, 3, 3, 1, 0),
    (1, 64, 73, 73, 80, 1, 1, 1, 0),
    (1, 80, 73, 73, 192, 3, 3, 1, 0),
    (2, 48, 35, 35, 64, 5, 5, 1, 2),
    (2, 192, 35, 35, 48, 1, 1, 1, 0),
    (1, 288, 35, 35, 384, 3, 3, 2, 0),
    (2, 128, 17, 17, 128, 1, 7, 1, 0),
    (2, 160, 17, 17, 192, 7, 1, 1, 3),
    (2, 768, 17, 17, 160, 1, 1, 1, 0),
    (2, 192, 17, 17, 320, 3, 3, 2, 0),
    (2, 384, 8, 8, 384, 1, 3, 1, 0),
    (2, 384, 8, 8, 384, 3, 1, 1, 1),
    (2, 2048, 8, 8, 448, 1, 1, 1, 0),
    (1, 3, 224, 224, 64, 3, 3, 1, 1),
    (1, 512, 14, 14, 512, 3, 3, 1, 1),
]


@pytest.mark.parametrize("case", NETWORK_LAYER_CASES)
def test_conv_nchw_network_layers(K, co, case):
    N, CI, H, W, CO, KH, KW, s, p = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, CI, H, W)).astype(np.float16)
    w = (rng.standard_normal((CO, CI, KH, KW)) / np.sqrt(CI * KH * KW)).astype(np.float16)
    want = co.conv2d_nchw(x, w, s, p, np.float16)
    out = poison(want.shape, torch.float16)
    K.conv2d_nchw(dev(x), dev(w), stride=s, padding=p, out=out)
    check(out, want, "network layer %s" % (case,))


def test_conv_nchw_int8_and_plan(K, co):
    rng = np.random.default_rng(12)
    x, w = rand_i8(rng, (2, 32, 10, 10), False), rand_i8(rng, (48, 32, 3, 3), True)
    want = co.conv2d_nchw(x, w, 1, 1)
    out = poison(want.shape, torch.int32)
    plan = K.plan_conv2d_nchw(dev(x), dev(w), stride=1, padding=1, out=out)
    plan.launch()
    check(out, want, "nchw int8")
    out.view(torch.uint8).fill_(0xCD)
    plan.launch()
    check(out, want, "nchw int8 relaunch")


def test_conv_nchw_int8_pointwise_in_place(K, co):
    rng = np.random.default_rng(31)
    for (N, CI, H, W, CO) in [(3, 64, 8, 8, 96), (2, 272, 4, 12, 40), (1, 128, 16, 16, 256)]:
        x, w = rand_i8(rng, (N, CI, H, W), False), rand_i8(rng, (CO, CI, 1, 1), True)
        check(K.conv2d_nchw(dev(x), dev(w)), co.conv2d_nchw(x, w, 1, 0), "nchw int8 1x1 %s" % ((N, CI, H, W, CO),))


@pytest.mark.parametrize("case", [(2, 3, 20, 20, 32, 7, 7, 2, 3), (2, 16, 9, 13, 32, 3, 3, 1, 1), (1, 5, 11, 11, 16, 3, 4, 1, 2)])
def test_conv_nchw_int8_few_channels(K, co, case):
    N, CI, H, W, CO, KH, KW, s, p = case
    rng = np.random.default_rng(sum(case))
    x, w = rand_i8(rng, (N, CI, H, W), False), rand_i8(rng, (CO, CI, KH, KW), True)
    out = K.conv2d_nchw(dev(x), dev(w), stride=s, padding=p)
    check(out, co.conv2d_nchw(x, w, s, p), "nchw int8 stem %s" % (case,))


@pytest.mark.parametrize("case", [(4, 512, 7, 7, 512, 3, 3, 1, 1), (2, 2048, 7, 7, 256, 1, 1, 1, 0), (8, 256, 14, 14, 64, 3, 3, 2, 1)])
def test_conv_nchw_small_output_long_reduction_splits_k(K, co, case):
    """Late-network shapes: few output tiles, thousands of reduction steps.  The plan cuts K into
    workspace slabs and a last kernel adds them in slab order: same bits on every launch, int8 exact."""
    N, CI, H, W, CO, KH, KW, s, p = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, CI, H, W)).astype(np.float16)
    w = (rng.standard_normal((CO, CI, KH, KW)) / np.sqrt(CI * KH * KW)).astype(np.float16)
    for od, tdt in ((np.float16, torch.float16), (np.float32, torch.float32)):
        want = co.conv2d_nchw(x, w, s, p, od)
        out = poison(want.shape, tdt)
        plan = K.plan_conv2d_nchw(dev(x), dev(w), stride=s, padding=p, out=out)
        assert plan.knobs()["split_k"] > 1, plan.knobs()
        plan.launch()
        check(out, want, "nchw split-K %s" % (case,))
        first = out.clone()
        out.view(torch.uint8).fill_(0xCD)
        plan.launch()
        assert torch.equal(out, first)
        off = poison(want.shape, tdt)
        K.conv2d_nchw(dev(x), dev(w), stride=s, padding=p, out=off, knobs=dict(split_k=1))
        check(off, want, "nchw, split-K off %s" % (case,))
    xi, wi = rand_i8(rng, (N, CI, H, W), False), rand_i8(rng, (CO, CI, KH, KW), True)
    plan = K.plan_conv2d_nchw(dev(xi), dev(wi), stride=s, padding=p)
    assert (plan.knobs()["split_k"] > 1) == (CI * KH * KW >= 4096), plan.knobs()  # half the K blocks in int8
    check(plan.launch(), co.conv2d_nchw(xi, wi, s, p), "nchw int8 split-K %s" % (case,))
    check(K.conv2d_nchw(dev(xi), dev(wi), stride=s, padding=p, knobs=dict(split_k=3)), co.conv2d_nchw(xi, wi, s, p),
          "nchw int8 split-K 3 %s" % (case,))


@pytest.mark.parametrize("case", [(4, 28, 28, 64, 64, 3, 3, 1, 1, 1, 0), (2, 14, 14, 256, 128, 3, 3, 1, 0, 1, 0),
                                  (3, 16, 16, 32, 48, 1, 1, 1, 0, 1, 0)])
def test_t2d_stride1_through_the_registry(K, co, case):
    """The reference's "transposed" conv at stride 1 against its own staging restated in numpy."""
    from heron_b200.ops import cuda as heron_cuda
    N, H, W, CI, CO, KH, KW, s, p, d, op_ = case
    t = _task(heron_cuda, "t2d", list(case) + ["float16", "float16"], "GPU_TENSOR_CORE")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, CI, H, W)).astype(np.float16)
    w = (rng.standard_normal((CO, CI, KH, KW)) / np.sqrt(CI * KH * KW)).astype(np.float16)
    want = npo.t2d_nchw_stride1(x, w, p, np.float16)
    assert tuple(args[-1].shape) == want.shape
    out = poison(want.shape, torch.float16)
    handle(dev(x), dev(w), out)
    check(out, want, "t2d %s" % (case,))


@pytest.mark.parametrize("case", [(2, 4, 14, 14, 64, 64, 3, 3, 3, 1, 1, 1), (2, 4, 12, 12, 32, 48, 1, 1, 1, 2, 0, 1),
                                  (1, 3, 9, 11, 16, 32, 2, 3, 1, (1, 2, 1), 1, 1), (2, 2, 8, 8, 64, 128, 1, 1, 1, 1, 0, 1),
                                  (1, 5, 6, 7, 3, 16, 3, 3, 3, 1, 1, 1)])
def test_conv3d_ncdhw(K, co, case):
    """(N, D, H, W, CI, CO, KD, KH, KW, stride, pad, dilation): the reference's c3d cases scaled
    down, unequal taps and strides, the 1x1x1 form that runs on the tensors in place, 3 channels."""
    from heron_b200.ops import cuda as heron_cuda
    N, D, H, W, CI, CO, KD, KH, KW, s, p, d = case
    rng = np.random.default_rng(sum(v if isinstance(v, int) else 5 for v in case))
    x = rng.standard_normal((N, CI, D, H, W)).astype(np.float16)
    w = (rng.standard_normal((CO, CI, KD, KH, KW)) / np.sqrt(CI * KD * KH * KW)).astype(np.float16)
    t = _task(heron_cuda, "c3d", list(case) + ["float16", "float16"], "GPU_TENSOR_CORE")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    want = co.conv3d_ncdhw(x, w, s, p, np.float16)
    assert tuple(args[-1].shape) == want.shape
    out = poison(want.shape, torch.float16)
    handle(dev(x), dev(w), out)
    check(out, want, "c3d fp16 %s %s" % (case, handle.knobs))
    check(K.conv3d_ncdhw(dev(x), dev(w), s, p), co.conv3d_ncdhw(x, w, s, p), "c3d fp32 out %s" % (case,))
    xi, wi = rand_i8(rng, (N, CI, D, H, W), False), rand_i8(rng, (CO, CI, KD, KH, KW), True)
    plan = K.plan_conv3d_ncdhw(dev(xi), dev(wi), s, p)
    check(plan.launch(), co.conv3d_ncdhw(xi, wi, s, p), "c3d int8 %s" % (case,))


def test_conv_nchw_through_the_registry(K, co):
    """`c2d` of the tensor-core registry, with a ResNet-50 table row scaled down in batch."""
    from heron_b200.ops import cuda as heron_cuda
    t = _task(heron_cuda, "c2d", [4, 28, 28, 128, 128, 3, 3, 1, 1, 1, "float16", "float16"], "GPU_TENSOR_CORE")
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    assert [a.shape for a in args] == [(4, 128, 28, 28), (128, 128, 3, 3), (4, 128, 28, 28)]
    rng = np.random.default_rng(3)
    x = rng.standard_normal(args[0].shape).astype(np.float16)
    w = (rng.standard_normal(args[1].shape) / 34.0).astype(np.float16)
    out = poison(args[2].shape, torch.float16)
    handle(dev(x), dev(w), out)
    check(out, co.conv2d_nchw(x, w, 1, 1, np.float16), "c2d registry")


def test_x86_batched_gemm_through_the_registry(K, co):
    from heron_b200.ops import x86 as heron_cpu
    t = _task(heron_cpu, "bmm", [3, 130, 64, 96, "float16", "float16"], "CPU")  # dtype arguments are ignored
    t.knob_manager.randSample()
    handle, args = t.instantiate(t.knob_manager)
    assert [a.dtype for a in args] == ["uint8", "int8", "int32"]
    rng = np.random.default_rng(31)
    a, b = rand_i8(rng, (3, 130, 64), False), rand_i8(rng, (3, 96, 64), True)
    out = poison(args[-1].shape, torch.int32)
    handle(dev(a), dev(b), out)
    check(out, co.bmm_int(a, b), "x86 bmm")


def test_bounded_wait_runs_out_cleanly(K, co):
    """Failure detection without a fault: a diagnostic launch whose producer warp stays silent, so
    the MMA and epilogue warps' bounded waits run out (0.1 s limit for this launch).  The kernel
    must return by itself, leave HB_ERR_TIMEOUT in the status word, free its TMEM and leave the
    context usable: the next launch on the same device is correct."""
    from heron_b200 import _lib
    rng = np.random.default_rng(1)
    a, b = rand_i8(rng, (256, 128), False), rand_i8(rng, (256, 128), True)
    ta, tb = dev(a), dev(b)
    out = poison((256, 256), torch.int32)
    K.gemm(ta, tb, out=out, knobs=dict(cta_group=1, silent_producer=1))
    assert _lib.last_status() == _lib.HB_ERR_TIMEOUT
    assert _lib.last_status() == 0  # reading clears it
    for _ in range(3):  # TMEM was released: full-size allocations succeed again
        K.gemm(ta, tb, out=out, knobs=dict(cta_group=1, tile_n=256))
        check(out, co.gemm_int(a, b), "after timeout")
    assert _lib.last_status() == 0


# ---- property tests over random small shapes ------------------------------------------------------
from hypothesis import HealthCheck, given, settings, strategies as st  # noqa: E402



def _props(examples):
    """Settings of the property tests. The examples are drawn from a fixed seed, so that a run of
    the suite is repeatable; HB_PROP_RANDOM=1 draws fresh ones and HB_PROP_SCALE=n draws n times as
    many, for a deeper search by hand."""
    scale = int(os.environ.get("HB_PROP_SCALE", "1"))
    return settings(max_examples=examples * scale, deadline=None, database=None,
                    derandomize=os.environ.get("HB_PROP_RANDOM", "0") != "1",
                    suppress_health_check=[HealthCheck.function_scoped_fixture])


_prop = _props(40)


@_prop
@given(M=st.integers(1, 300), N=st.integers(1, 300), K16=st.integers(1, 20), a_signed=st.booleans(),
       cta_group=st.sampled_from([0, 1, 2]), seed=st.integers(0, 2 ** 20))
def test_gemm_int8_random_shapes(K, co, M, N, K16, a_signed, cta_group, seed):
    """Any M, any N (rows that are not 16-byte multiples take the direct-store epilogue), K a
    multiple of 16 bytes."""
    rng = np.random.default_rng(seed)
    a, b = rand_i8(rng, (M, 16 * K16), a_signed), rand_i8(rng, (N, 16 * K16), True)
    check(k_gemm(K, a, b, knobs=dict(cta_group=cta_group)), co.gemm_int(a, b), "gemm %s" % ((M, N, 16 * K16),))


@_prop
@given(B=st.integers(1, 5), M=st.integers(1, 200), N=st.integers(1, 40), K8=st.integers(1, 12),
       seed=st.integers(0, 2 ** 20))
def test_bmm_fp16_random_shapes(K, co, B, M, N, K8, seed):
    rng = np.random.default_rng(seed)
    Kd = 8 * K8
    a = (rng.standard_normal((B, M, Kd)) / np.sqrt(Kd)).astype(np.float16)
    b = rng.standard_normal((B, 4 * N, Kd)).astype(np.float16)
    check(k_bmm(K, a, b), co.bmm_f16(a, b), "bmm %s" % ((B, M, 4 * N, Kd),))


@_prop
@given(N=st.integers(1, 4), H=st.integers(1, 20), W=st.integers(1, 20), CI=st.sampled_from([32, 64, 96]),
       CO16=st.integers(1, 6), KH=st.integers(1, 5), KW=st.integers(1, 5), sh=st.integers(1, 3), sw=st.integers(1, 3),
       pad=st.integers(0, 3), dil=st.integers(1, 2), algo=st.sampled_from([0, 1]), seed=st.integers(0, 2 ** 20))
def test_conv_int8_random_geometry(K, co, N, H, W, CI, CO16, KH, KW, sh, sw, pad, dil, algo, seed):
    """Strides, paddings, dilations and window sizes at random, including windows larger than the
    image plus padding (rejected) and one-pixel outputs."""
    span_h, span_w = (KH - 1) * dil + 1, (KW - 1) * dil + 1
    rng = np.random.default_rng(seed)
    x, w = rand_i8(rng, (N, H, W, CI), False), rand_i8(rng, (KH, KW, CI, 16 * CO16), True)
    if H + 2 * pad < span_h or W + 2 * pad < span_w:
        from heron_b200._lib import HB_ERR_SHAPE, HeronB200Error
        with pytest.raises(HeronB200Error) as e:
            K.conv2d_nhwc(dev(x), dev(w), (sh, sw), pad, dil)
        assert e.value.status == HB_ERR_SHAPE
        return
    got = k_conv(K, x, w, (sh, sw), pad, dil, knobs=dict(conv_algo=algo))
    check(got, co.conv2d_nhwc_int(x, w, (sh, sw), pad, dil), "conv %s" % ((N, H, W, CI, 16 * CO16, KH, KW, sh, sw, pad, dil),))


@_prop
@given(N=st.integers(1, 3), H=st.integers(1, 40), W=st.integers(1, 40), CO=st.sampled_from([64, 128]),
       KH=st.integers(1, 3), KW=st.integers(1, 3), pad=st.integers(0, 2), dil=st.integers(1, 2),
       half_out=st.booleans(), seed=st.integers(0, 2 ** 20))
def test_conv_strip_random_geometry(K, co, N, H, W, CO, KH, KW, pad, dil, half_out, seed):
    """The strip kernel over random stride-1 geometries: ragged last row groups, windows that
    overhang the padding, one-row images, dilation."""
    if H + 2 * pad < (KH - 1) * dil + 1 or W + 2 * pad < (KW - 1) * dil + 1:
        return
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, H, W, 64)).astype(np.float16)
    w = (rng.standard_normal((KH, KW, 64, CO)) / np.sqrt(KH * KW * 64)).astype(np.float16)
    od = np.float16 if half_out else np.float32
    got = k_conv(K, x, w, 1, pad, dil, out_dtype=od, knobs=dict(conv_algo=2))
    check(got, co.conv2d_nhwc_f16(x, w, 1, pad, dil, od), "strip %s" % ((N, H, W, CO, KH, KW, pad, dil),))


@_props(80)
@given(N=st.integers(1, 4), CI=st.sampled_from([1, 3, 4, 8, 16, 24, 64, 72, 136]), H=st.integers(1, 24),
       W=st.integers(1, 24), CO8=st.integers(1, 12), KH=st.integers(1, 7), KW=st.integers(1, 8),
       sh=st.integers(1, 3), sw=st.integers(1, 3), pad=st.integers(0, 3), int8=st.booleans(),
       half_out=st.booleans(), split_k=st.sampled_from([0, 0, 1, 3]), seed=st.integers(0, 2 ** 20))
def test_conv_nchw_random_geometry(K, co, N, CI, H, W, CO8, KH, KW, sh, sw, pad, int8, half_out, split_k, seed):
    """The NCHW operator over random geometries, so that every route it can take is hit: tensors
    in place (1x1, 16-byte rows), the few-channel form, kept-pixel glue for strided 1x1, the tile
    transposes with and without 8-byte accesses, the strip kernel, workspace split-K."""
    if H + 2 * pad < KH or W + 2 * pad < KW:
        return
    rng = np.random.default_rng(seed)
    CO = 8 * CO8 * (2 if int8 else 1)  # output rows of the filter matrix are 16-byte multiples
    if int8:
        x, w = rand_i8(rng, (N, CI, H, W), False), rand_i8(rng, (CO, CI, KH, KW), True)
        od = None
    else:
        x = rng.standard_normal((N, CI, H, W)).astype(np.float16)
        w = (rng.standard_normal((CO, CI, KH, KW)) / np.sqrt(CI * KH * KW)).astype(np.float16)
        od = np.float16 if half_out else np.float32
    want = co.conv2d_nchw(x, w, (sh, sw), pad, od)
    out = poison(want.shape, _T[want.dtype])
    K.conv2d_nchw(dev(x), dev(w), stride=(sh, sw), padding=pad, out=out, knobs=dict(split_k=split_k))
    check(out, want, "nchw %s" % ((N, CI, H, W, CO, KH, KW, sh, sw, pad, int8, half_out, split_k),))


@_prop
@given(N=st.integers(1, 2), CI=st.sampled_from([3, 16, 40]), D=st.integers(1, 6), H=st.integers(1, 10),
       W=st.integers(1, 10), CO8=st.integers(1, 6), KD=st.integers(1, 3), KH=st.integers(1, 3), KW=st.integers(1, 3),
       sd=st.integers(1, 2), sh=st.integers(1, 2), sw=st.integers(1, 3), pad=st.integers(0, 2), int8=st.booleans(),
       seed=st.integers(0, 2 ** 20))
def test_conv3d_random_geometry(K, co, N, CI, D, H, W, CO8, KD, KH, KW, sd, sh, sw, pad, int8, seed):
    if D + 2 * pad < KD or H + 2 * pad < KH or W + 2 * pad < KW:
        return
    rng = np.random.default_rng(seed)
    CO = 8 * CO8 * (2 if int8 else 1)
    if int8:
        x, w = rand_i8(rng, (N, CI, D, H, W), False), rand_i8(rng, (CO, CI, KD, KH, KW), True)
    else:
        x = rng.standard_normal((N, CI, D, H, W)).astype(np.float16)
        w = (rng.standard_normal((CO, CI, KD, KH, KW)) / np.sqrt(CI * KD * KH * KW)).astype(np.float16)
    want = co.conv3d_ncdhw(x, w, (sd, sh, sw), pad)
    got = K.conv3d_ncdhw(dev(x), dev(w), (sd, sh, sw), pad)
    check(got, want, "c3d %s" % ((N, CI, D, H, W, CO, KD, KH, KW, sd, sh, sw, pad, int8),))


def test_further_outputs_of_a_plan(K, co):
    """hb_plan_set_peer_outputs on one GPU: every tile goes to the plan's output and to each
    further output (here ordinary buffers of the same device; across GPUs they are the other
    ranks' buffers, tests/multi_rank_check.py).  GEMM in CTA pairs with a ragged edge, a batched
    GEMM with eight epilogue warps, an fp16 conv through im2col loads; taking the outputs away
    again; the refusals."""
    from heron_b200._lib import HB_ERR_KNOB, HeronB200Error
    rng = np.random.default_rng(99)
    a, b = rand_i8(rng, (520, 1152), False), rand_i8(rng, (328, 1152), True)
    out = poison((520, 328), torch.int32)
    extra = [poison((520, 328), torch.int32) for _ in range(3)]
    plan = K.plan_gemm(dev(a), dev(b), out=out, knobs=dict(cta_group=2))
    plan.set_peer_outputs(extra)
    plan.launch()
    want = co.gemm_int(a, b)
    for t in [out] + extra:
        check(t, want, "gemm, further outputs")
    for t in extra:
        t.fill_(-7)
    plan.set_peer_outputs([])
    out.fill_(0)
    plan.launch()
    check(out, want, "gemm, outputs removed")
    assert all(bool((t == -7).all()) for t in extra)

    a3, b3 = rand_i8(rng, (5, 200, 64), True), rand_i8(rng, (5, 264, 64), True)
    out3 = poison((5, 200, 264), torch.int32)
    more = [poison((5, 200, 264), torch.int32) for _ in range(2)]
    plan3 = K.plan_bmm(dev(a3), dev(b3), out=out3, knobs=dict(epi_warps=8))
    plan3.set_peer_outputs(more)
    plan3.launch()
    for t in [out3] + more:
        check(t, co.bmm_int(a3, b3), "bmm, further outputs")

    x = rng.standard_normal((3, 9, 11, 64)).astype(np.float16)
    w = (rng.standard_normal((3, 3, 64, 128)) / 24.0).astype(np.float16)
    outc = poison((3, 9, 11, 128), torch.float16)
    morec = [poison((3, 9, 11, 128), torch.float16)]
    planc = K.plan_conv2d_nhwc(dev(x), dev(w), 1, 1, 1, out=outc, knobs=dict(conv_algo=1))
    planc.set_peer_outputs(morec)
    planc.launch()
    for t in [outc] + morec:
        check(t, co.conv2d_nhwc_f16(x, w, 1, 1, 1, np.float16), "conv, further outputs")

    for knobs in (dict(conv_algo=1, epilogue=2), dict(conv_algo=2), dict(conv_algo=1, split_k=2)):
        p2 = K.plan_conv2d_nhwc(dev(x), dev(w), 1, 1, 1, out_dtype=torch.float32, knobs=knobs)
        with pytest.raises(HeronB200Error) as e:
            p2.set_peer_outputs([torch.empty_like(p2.out)])
        assert e.value.status == HB_ERR_KNOB
    with pytest.raises(ValueError):
        plan.set_peer_outputs([torch.empty((520, 320), dtype=torch.int32, device="cuda")])
