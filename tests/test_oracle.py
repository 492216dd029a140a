"""The oracle against itself: C restatement vs numpy restatement vs the committed golden cases,
plus the timed CPU baseline against both.  CPU only."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from golden_util import assert_matches, load_cases, run_case
from oracle import np_oracle as npo


@pytest.fixture(scope="module")
def co(oracle_libs):
    from oracle import c_oracle
    return c_oracle


@pytest.fixture(scope="module")
def dl(oracle_libs):
    from oracle import dlboost
    return dlboost


def test_golden_numpy():
    for name, case in load_cases().items():
        got = run_case(name, case, npo.gemm_int, npo.bmm_int, npo.gemm_f16, npo.conv2d_nhwc_int,
                       npo.conv2d_nhwc_f16, npo.conv2d_nhwc_packed)
        assert_matches(name, got, case["out"])


def test_golden_c(co):
    for name, case in load_cases().items():
        got = run_case(name, case, co.gemm_int, co.bmm_int, co.gemm_f16, co.conv2d_nhwc_int,
                       co.conv2d_nhwc_f16, co.conv2d_nhwc_packed)
        assert_matches(name, got, case["out"])


def test_golden_neighbour_cases_both_oracles(co):
    from golden_util import run_neighbour_case
    for name, case in load_cases("kat_neighbours.npz").items():
        for impl in (npo, co):
            got = run_neighbour_case(name, case, impl.gemv, impl.conv1d_ncw, impl.conv1d_nwc_packed)
            assert_matches(name, got, case["out"])


def test_golden_fp16_cases_bit_exact_between_oracles(co):
    """Both restatements accumulate in double, so even the floating-point cases agree to the bit."""
    for name, case in load_cases().items():
        if "f16" not in name:
            continue
        a = run_case(name, case, None, None, npo.gemm_f16, None, npo.conv2d_nhwc_f16, None)
        b = run_case(name, case, None, None, co.gemm_f16, None, co.conv2d_nhwc_f16, None)
        assert np.array_equal(a.view(np.uint16 if a.dtype == np.float16 else np.uint32),
                              b.view(np.uint16 if b.dtype == np.float16 else np.uint32)), name


@settings(max_examples=40, deadline=None)
@given(M=st.integers(1, 40), K=st.integers(1, 70), N=st.integers(1, 40), a_signed=st.booleans(),
       b_signed=st.booleans(), seed=st.integers(0, 2 ** 31))
def test_gemm_int_c_vs_numpy(co, M, K, N, a_signed, b_signed, seed):
    rng = np.random.default_rng(seed)
    a = rng.integers(-128, 128, (M, K)).astype(np.int8) if a_signed else rng.integers(0, 256, (M, K), dtype=np.uint8)
    b = rng.integers(-128, 128, (N, K)).astype(np.int8) if b_signed else rng.integers(0, 256, (N, K), dtype=np.uint8)
    assert np.array_equal(co.gemm_int(a, b), npo.gemm_int(a, b))


@settings(max_examples=40, deadline=None)
@given(N=st.integers(1, 3), H=st.integers(1, 9), W=st.integers(1, 9), CI=st.sampled_from([4, 8, 16]),
       CO=st.sampled_from([1, 8, 32]), KH=st.integers(1, 3), KW=st.integers(1, 3),
       stride=st.integers(1, 3), pad=st.integers(0, 2), dil=st.integers(1, 2),
       seed=st.integers(0, 2 ** 31))
def test_conv_int_c_vs_numpy(co, N, H, W, CI, CO, KH, KW, stride, pad, dil, seed):
    if H + 2 * pad < (KH - 1) * dil + 1 or W + 2 * pad < (KW - 1) * dil + 1:
        return
    rng = np.random.default_rng(seed)
    x = rng.integers(0, 256, (N, H, W, CI), dtype=np.uint8)
    w = rng.integers(-128, 128, (KH, KW, CI, CO)).astype(np.int8)
    assert np.array_equal(co.conv2d_nhwc_int(x, w, stride, pad, dil), npo.conv2d_nhwc_int(x, w, stride, pad, dil))


def test_conv_against_scipy_correlate():
    """A third, library implementation of the same sum: per-channel 2-D cross-correlation."""
    from scipy.signal import correlate2d
    rng = np.random.default_rng(5)
    x = rng.integers(0, 256, (1, 6, 7, 3), dtype=np.uint8)
    w = rng.integers(-128, 128, (3, 3, 3, 2)).astype(np.int8)
    want = np.zeros((1, 6, 7, 2), dtype=np.int64)
    for f in range(2):
        for c in range(3):
            want[0, :, :, f] += correlate2d(x[0, :, :, c].astype(np.int64), w[:, :, c, f].astype(np.int64),
                                            mode="same")
    assert np.array_equal(npo.conv2d_nhwc_int(x, w, 1, 1, 1), want.astype(np.int32))


def test_fp16_paths(co):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((33, 130)).astype(np.float16)
    b = rng.standard_normal((17, 130)).astype(np.float16)
    assert np.array_equal(co.gemm_f16(a, b), npo.gemm_f16(a, b))
    x = rng.standard_normal((2, 8, 5, 16)).astype(np.float16)
    w = rng.standard_normal((3, 3, 16, 24)).astype(np.float16)
    for out_dtype in (np.float32, np.float16):
        assert np.array_equal(co.conv2d_nhwc_f16(x, w, (2, 1), 1, 1, out_dtype),
                              npo.conv2d_nhwc_f16(x, w, (2, 1), 1, 1, out_dtype))


def test_half_conversion_matches_numpy(co):
    L = co.lib()
    halves = np.arange(0, 65536, 13, dtype=np.uint16)
    floats = halves.view(np.float16).astype(np.float32)
    for h, f in zip(halves.tolist(), floats.tolist()):
        got = L.oracle_half_to_float(h)
        assert (np.isnan(got) and np.isnan(f)) or got == f
    rng = np.random.default_rng(11)
    vals = (rng.standard_normal(4000) * rng.choice([1e-8, 1e-5, 1e-2, 1.0, 300.0, 6e4], 4000)).astype(np.float32)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    for v, w in zip(vals.tolist(), want.tolist()):
        assert L.oracle_float_to_half(v) == w


def test_empty_and_degenerate(co):
    a = np.zeros((0, 8), dtype=np.uint8)
    b = np.zeros((4, 8), dtype=np.int8)
    assert co.gemm_int(a, b).shape == (0, 4) and npo.gemm_int(a, b).shape == (0, 4)
    # a 1x1 window with stride 2 on a 1-pixel image
    x = np.full((1, 1, 1, 4), 3, dtype=np.uint8)
    w = np.full((1, 1, 4, 2), -2, dtype=np.int8)
    assert np.array_equal(co.conv2d_nhwc_int(x, w, 2, 0, 1), np.full((1, 1, 1, 2), -24, dtype=np.int32))


def test_filter_packing_roundtrip():
    rng = np.random.default_rng(2)
    w = rng.integers(-128, 128, (3, 3, 16, 96)).astype(np.int8)
    for sco in (32, 48):
        wp = npo.pack_filter_x86(w, sco)
        assert wp.shape == (96 // sco, 3, 3, 4, sco, 4)
        assert np.array_equal(npo.unpack_filter_x86(wp), w)


def test_cpu_baseline_matches_oracle(dl):
    """The timed DL Boost port computes what the oracle computes (VNNI path or its scalar twin)."""
    rng = np.random.default_rng(9)
    a = rng.integers(0, 256, (70, 64), dtype=np.uint8)
    b = rng.integers(-128, 128, (48, 64)).astype(np.int8)
    assert np.array_equal(dl.GemmU8S8(70, 64, 48)(a, b), npo.gemm_int(a, b))
    a = rng.integers(-128, 128, (3, 33, 64)).astype(np.int8)
    b = rng.integers(-128, 128, (3, 32, 64)).astype(np.int8)
    assert np.array_equal(dl.BmmS8S8(3, 33, 64, 32)(a, b), npo.bmm_int(a, b))
    x = rng.integers(0, 256, (3, 7, 7, 64), dtype=np.uint8)
    w = rng.integers(-128, 128, (3, 3, 64, 192)).astype(np.int8)
    for sco in (64, 48, 32):
        wp = npo.pack_filter_x86(w, sco)
        assert np.array_equal(dl.ConvPacked(3, 7, 7, 64, 192, 3, 3, 1, 1, 1, sco)(x, wp),
                              npo.conv2d_nhwc_packed(x, wp, 1, 1, 1))
    af = rng.standard_normal((37, 100)).astype(np.float16)
    bf = rng.standard_normal((19, 100)).astype(np.float16)
    if dl.has_avx512():
        got = dl.GemmF16(37, 100, 19)(af, bf)
        want = npo.gemm_f16(af, bf)
        assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()


def test_nchw_operator_three_ways(co):
    """The NCHW operator: the reference's im2col formulation (numpy), the direct sum (C), and the
    NHWC restatement on transposed tensors all agree to the bit."""
    rng = np.random.default_rng(21)
    for (N, CI, H, W, CO, KH, KW, s, p) in [(2, 3, 9, 9, 8, 7, 7, 2, 3), (1, 16, 6, 7, 5, 3, 3, 1, 1),
                                            (2, 32, 5, 5, 16, 1, 1, 2, 0)]:
        x = rng.integers(0, 256, (N, CI, H, W), dtype=np.uint8)
        w = rng.integers(-128, 128, (CO, CI, KH, KW)).astype(np.int8)
        a = npo.conv2d_nchw_int(x, w, s, p)
        b = co.conv2d_nchw(x, w, s, p)
        c = npo.conv2d_nhwc_int(np.ascontiguousarray(x.transpose(0, 2, 3, 1)),
                                np.ascontiguousarray(w.transpose(2, 3, 1, 0)), s, p, 1).transpose(0, 3, 1, 2)
        assert np.array_equal(a, b) and np.array_equal(a, c)
        xf = rng.standard_normal((N, CI, H, W)).astype(np.float16)
        wf = rng.standard_normal((CO, CI, KH, KW)).astype(np.float16)
        for od in (np.float32, np.float16):
            assert np.array_equal(npo.conv2d_nchw_f16(xf, wf, s, p, od), co.conv2d_nchw(xf, wf, s, p, od))


def test_conv3d_c_vs_numpy(co):
    rng = np.random.default_rng(303)
    for (N, CI, D, H, W, CO, KD, KH, KW, s, p) in [(2, 4, 3, 5, 6, 8, 3, 3, 3, 1, 1), (1, 8, 4, 6, 5, 8, 1, 1, 1, 2, 0),
                                                  (2, 3, 5, 4, 7, 8, 2, 3, 1, (2, 1, 2), 1), (1, 4, 2, 3, 3, 8, 3, 3, 3, 1, 1)]:
        x = rng.integers(-128, 128, (N, CI, D, H, W)).astype(np.int8)
        w = rng.integers(-128, 128, (CO, CI, KD, KH, KW)).astype(np.int8)
        assert np.array_equal(co.conv3d_ncdhw(x, w, s, p), npo.conv3d_ncdhw(x, w, s, p))
        xf = rng.standard_normal((N, CI, D, H, W)).astype(np.float16)
        wf = rng.standard_normal((CO, CI, KD, KH, KW)).astype(np.float16)
        assert np.array_equal(co.conv3d_ncdhw(xf, wf, s, p), npo.conv3d_ncdhw(xf, wf, s, p))
    # depth 1, one depth tap: the 2-D operator
    x = rng.integers(0, 256, (2, 4, 1, 6, 6), dtype=np.uint8)
    w = rng.integers(-128, 128, (8, 4, 1, 3, 3)).astype(np.int8)
    assert np.array_equal(co.conv3d_ncdhw(x, w, 1, 0)[:, :, 0], co.conv2d_nchw(x[:, :, 0], w[:, :, 0], 1, 0))


def test_t2d_stride1_is_the_padded_conv(co):
    """The reference's transposed-conv expression at stride 1, staged as it stages it, against the
    C conv loops with padding K-1-p."""
    rng = np.random.default_rng(77)
    for (N, CI, H, W, CO, K, p) in [(2, 8, 6, 7, 16, 3, 1), (1, 4, 5, 5, 8, 3, 0), (2, 16, 9, 4, 8, 1, 0), (1, 8, 6, 6, 8, 5, 2)]:
        x = rng.integers(-128, 128, (N, CI, H, W)).astype(np.int8)
        w = rng.integers(-128, 128, (CO, CI, K, K)).astype(np.int8)
        want = npo.t2d_nchw_stride1(x, w, p)
        assert want.shape == (N, CO, H - 2 * p + K - 1, W - 2 * p + K - 1)
        assert np.array_equal(co.conv2d_nchw(x, w, 1, K - 1 - p), want)


def test_neighbour_operators_c_vs_numpy(co):
    """gemv and the two 1-D convolutions: the scalar C loops against the numpy restatement of the
    reference's own lowering (padded vector, explicit im2col, packed filter)."""
    rng = np.random.default_rng(404)
    a = rng.integers(0, 256, (37, 48), dtype=np.uint8)
    x = rng.integers(-128, 128, (1, 48)).astype(np.int8)
    got = co.gemv(a, x)
    assert np.array_equal(got, npo.gemv(a, x)) and not got[:, 1:].any()
    assert np.array_equal(got[:, 0], a.astype(np.int64) @ x[0].astype(np.int64))
    ah = rng.standard_normal((20, 32)).astype(np.float16)
    xh = rng.standard_normal((1, 32)).astype(np.float16)
    assert np.array_equal(co.gemv(ah, xh), npo.gemv(ah, xh))
    assert np.array_equal(co.gemv(ah, xh, np.float16), npo.gemv(ah, xh, np.float16))
    # scan: the product with the constant triangle is an exclusive running sum
    a = rng.integers(0, 256, (9, 40), dtype=np.uint8)
    for N in (1, 17, 40, 55):
        got = co.scan(a, N)
        assert np.array_equal(got, npo.scan(a, N))
        run = np.concatenate([np.zeros((9, 1), np.int64), np.cumsum(a.astype(np.int64), axis=1)], axis=1)
        want = run[:, np.minimum(np.arange(N), 40)]
        assert np.array_equal(got, want)
    ah = rng.standard_normal((6, 24)).astype(np.float16)
    assert np.array_equal(co.scan(ah, 30), npo.scan(ah, 30))
    assert np.array_equal(co.scan(ah, 30, np.float16), npo.scan(ah, 30, np.float16))
    for (N, W, CI, CO, KW, s, p) in [(2, 19, 16, 24, 3, 1, 4), (3, 30, 8, 16, 1, 2, 0), (1, 12, 4, 8, 5, 3, 2)]:
        xi = rng.integers(-128, 128, (N, CI, W)).astype(np.int8)
        wi = rng.integers(-128, 128, (CO, CI, KW)).astype(np.int8)
        assert np.array_equal(co.conv1d_ncw(xi, wi, s, p), npo.conv1d_ncw(xi, wi, s, p))
        xf = rng.standard_normal((N, CI, W)).astype(np.float16)
        wf = rng.standard_normal((CO, CI, KW)).astype(np.float16)
        assert np.array_equal(co.conv1d_ncw(xf, wf, s, p), npo.conv1d_ncw(xf, wf, s, p))
        assert co.conv1d_ncw(xf, wf, s, p).shape == (N, CO, (W - KW + 2 * p) // s + 1)
    for (N, W, CI, CO, KW, s, p, d, sco) in [(2, 21, 8, 64, 3, 1, 4, 2, 64), (1, 17, 12, 96, 3, 2, 1, 1, 48), (2, 9, 4, 32, 1, 1, 0, 1, 32)]:
        xi = rng.integers(0, 256, (N, W, CI), dtype=np.uint8)
        w = rng.integers(-128, 128, (KW, CI, CO)).astype(np.int8)
        wp = npo.pack_filter_x86_1d(w, sco)
        assert wp.shape == (CO // sco, KW, CI // 4, sco, 4)
        got = co.conv1d_nwc_packed(xi, wp, s, p, d)
        assert np.array_equal(got, npo.conv1d_nwc_packed(xi, wp, s, p, d))
        WO = (W - ((KW - 1) * d + 1) + 2 * p) // s + 1
        assert got.shape == (N, WO, CO // sco, sco)
        # one element by hand
        n, q, f = N - 1, WO // 2, CO - 1
        want = 0
        for rx in range(KW):
            xw = q * s + rx * d - p
            if 0 <= xw < W:
                want += int(xi[n, xw].astype(np.int64) @ w[rx, :, f].astype(np.int64))
        assert int(got[n, q, f // sco, f % sco]) == want
