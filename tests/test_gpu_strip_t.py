"""The wide strip conv kernel (conv_algo 3: output channels on the MMA's M axis, 256 consecutive
output positions on N) against the oracle, through the C ABI, on a B200.  fp16 inputs, fp32
accumulation; the per-element and largest-error bounds of tests/test_gpu_parity.py."""
import numpy as np
import pytest
import torch

from test_gpu_parity import K, check, co, dev, k_conv, poison  # noqa: F401  (fixtures and helpers)

pytestmark = pytest.mark.gpu

WIDE_CASES = [
    # N, H, W, CI, CO, KH, KW, pad, dil   (stride 1, CO 64 or 128)
    (2, 8, 8, 64, 64, 3, 3, 1, 1),
    (8, 56, 56, 64, 64, 3, 3, 1, 1),
    (2, 12, 12, 64, 64, 3, 3, 0, 1),
    (1, 100, 100, 64, 64, 1, 1, 0, 1),
    (3, 13, 9, 64, 128, 2, 2, 1, 2),
    (2, 57, 31, 128, 64, 3, 1, 1, 1),
    (2, 126, 5, 64, 64, 3, 3, 1, 1),
    (2, 20, 100, 64, 64, 3, 3, 1, 1),
    (5, 28, 28, 64, 128, 3, 3, 1, 1),
    (1, 3, 3, 64, 64, 3, 3, 1, 1),
    (4, 7, 7, 64, 128, 1, 1, 0, 1),
]


@pytest.fixture(autouse=True)
def _status_clean(hb_lib):
    yield
    from heron_b200 import _lib
    assert _lib.last_status() == 0, "a bounded device-side wait ran out"


@pytest.mark.parametrize("case", WIDE_CASES)
def test_wide_strip_conv_fp16(K, co, case):
    N, H, W, CI, CO, KH, KW, p, d = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, H, W, CI)).astype(np.float16)
    w = (rng.standard_normal((KH, KW, CI, CO)) / np.sqrt(KH * KW * CI)).astype(np.float16)
    # (a 3x3 filter over 128 output channels leaves no room for the staging buffers of fp32 pixels)
    for od in ((np.float16,) if KH * KW * CI * CO * 2 > 140000 else (np.float32, np.float16)):
        want = co.conv2d_nhwc_f16(x, w, 1, p, d, od)
        check(k_conv(K, x, w, 1, p, d, out_dtype=od, knobs=dict(conv_algo=3)), want, "wide strip %s" % (case,))


from hypothesis import HealthCheck, given, settings, strategies as st


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck))
@given(N=st.integers(1, 3), H=st.integers(1, 40), W=st.integers(1, 60), CO=st.sampled_from([64, 128]),
       CI=st.sampled_from([64, 128]), KH=st.integers(1, 3), KW=st.integers(1, 3), pad=st.integers(0, 2),
       dil=st.integers(1, 2), half_out=st.booleans(), tile_n=st.sampled_from([0, 64, 128, 192, 256]),
       max_ctas=st.sampled_from([0, 1, 3]), seed=st.integers(0, 2 ** 20))
def test_wide_strip_random_geometry(K, co, N, H, W, CO, CI, KH, KW, pad, dil, half_out, tile_n, max_ctas, seed):
    """Random stride-1 geometries: tiles that start mid-row, short last tiles, windows that overhang
    the padding, one-row and one-column images, dilation, several tile widths, few CTAs."""
    from heron_b200._lib import HB_ERR_KNOB, HeronB200Error
    if H + 2 * pad < (KH - 1) * dil + 1 or W + 2 * pad < (KW - 1) * dil + 1:
        return
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, H, W, CI)).astype(np.float16)
    w = (rng.standard_normal((KH, KW, CI, CO)) / np.sqrt(KH * KW * CI)).astype(np.float16)
    od = np.float16 if half_out else np.float32
    try:
        got = k_conv(K, x, w, 1, pad, dil, out_dtype=od, knobs=dict(conv_algo=3, tile_n=tile_n, max_ctas=max_ctas))
    except HeronB200Error as e:
        assert e.status == HB_ERR_KNOB  # filter + two strips + one output tile beyond shared memory
        assert KH * KW * CI * CO * 2 + CI * 2 * 2 * 64 * 128 // 128 > 60000
        return
    check(got, co.conv2d_nhwc_f16(x, w, 1, pad, dil, od), "wide strip %s" % ((N, H, W, CI, CO, KH, KW, pad, dil, tile_n),))


def test_wide_strip_conv_one_hot_channels(K, co):
    """Every (input channel, output channel) pair lands where it should: a filter that is one-hot
    per tap maps input channel c of the tap's pixel to output channel (c * 7 + tap) % 64."""
    rng = np.random.default_rng(3)
    x = rng.integers(-4, 5, (2, 9, 10, 64)).astype(np.float16)
    w = np.zeros((3, 3, 64, 64), np.float16)
    for tap in range(9):
        for c in range(64):
            w[tap // 3, tap % 3, c, (c * 7 + tap) % 64] = 1.0
    got = k_conv(K, x, w, 1, 1, 1, out_dtype=np.float32, knobs=dict(conv_algo=3)).cpu().numpy()
    assert np.array_equal(got, co.conv2d_nhwc_f16(x, w, 1, 1, 1, np.float32))  # small integers: exact


def test_wide_strip_walks_its_ring_and_relaunches(K, co):
    """One CTA takes every tile in turn (ring and accumulator buffers reused many times); a second
    launch of the same plan gives the same bits."""
    rng = np.random.default_rng(11)
    x = rng.standard_normal((6, 30, 30, 64)).astype(np.float16)
    w = (rng.standard_normal((3, 3, 64, 64)) / 24.0).astype(np.float16)
    out = poison((6, 30, 30, 64), torch.float16)
    plan = K.plan_conv2d_nhwc(dev(x), dev(w), stride=1, padding=1, dilation=1, out=out,
                              knobs=dict(conv_algo=3, max_ctas=1))
    kn = plan.knobs()
    assert kn["conv_algo"] == 3 and kn["grid"] == 1, kn
    plan.launch()
    check(out, co.conv2d_nhwc_f16(x, w, 1, 1, 1, np.float16), "wide strip, one CTA")
    first = out.clone()
    out.view(torch.uint8).fill_(0xCD)
    plan.launch()
    assert torch.equal(out, first)


def test_wide_strip_refused_where_it_does_not_apply(K):
    from heron_b200._lib import HB_ERR_KNOB, HeronB200Error
    x = torch.zeros(2, 14, 14, 64, dtype=torch.float16, device="cuda")
    for w in (torch.zeros(3, 3, 64, 96, dtype=torch.float16, device="cuda"),     # CO not 64 or 128
              torch.zeros(5, 5, 64, 128, dtype=torch.float16, device="cuda")):   # 400 KiB filter
        with pytest.raises(HeronB200Error) as e:
            K.conv2d_nhwc(x, w, 1, 2, 1, knobs=dict(conv_algo=3))
        assert e.value.status == HB_ERR_KNOB
    w = torch.zeros(3, 3, 64, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(HeronB200Error) as e:
        K.conv2d_nhwc(x, w, 2, 1, 1, knobs=dict(conv_algo=3))  # stride 2
    assert e.value.status == HB_ERR_KNOB
    xi = torch.zeros(2, 14, 14, 128, dtype=torch.uint8, device="cuda")
    wi = torch.zeros(3, 3, 128, 64, dtype=torch.int8, device="cuda")
    with pytest.raises(HeronB200Error) as e:
        K.conv2d_nhwc(xi, wi, 1, 1, 1, knobs=dict(conv_algo=3))  # integer operands
    assert e.value.status == HB_ERR_KNOB


def test_cfg3_full_size_on_the_wide_strip_kernel(K, co):
    from heron_b200.workloads import make_inputs
    x, w = make_inputs("cfg3_conv_f16_resnet_s2")
    out = k_conv(K, x, w, 1, 1, 1, out_dtype=np.float16, knobs=dict(conv_algo=3))
    for n in (0, 13, 31):
        check(out[n:n + 1], co.conv2d_nhwc_f16(x[n:n + 1], w, 1, 1, 1, np.float16), "cfg3 image %d" % n)
    got = out.cpu().numpy().astype(np.float64).sum(axis=3)
    wsum = w.astype(np.float64).sum(axis=3, keepdims=True)
    xp = np.pad(x.astype(np.float64), ((0, 0), (1, 1), (1, 1), (0, 0)))
    want = np.zeros(got.shape)
    for ry in range(3):
        for rx in range(3):
            want += (xp[:, ry:ry + 56, rx:rx + 56, :] * wsum[ry, rx, :, 0]).sum(axis=3)
    assert np.abs(got - want).max() <= 64 * 2e-3 * np.abs(out.cpu().numpy().astype(np.float64)).max()
