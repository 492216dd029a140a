"""The strip conv kernel's fused-row form (conv_algo 4: pixels on the MMA's M axis, the three taps of
a filter row side by side on N, the epilogue adding the column groups shifted by one and two
pixels) against the oracle, through the C ABI, on a B200.  fp16 inputs, fp32 accumulation; the
per-element and largest-error bounds of tests/test_gpu_parity.py."""
import numpy as np
import pytest
import torch

from test_gpu_parity import K, check, co, dev, k_conv, poison  # noqa: F401  (fixtures and helpers)

pytestmark = pytest.mark.gpu

FUSED_CASES = [
    # N, H, W, CI, KH, pad, dil_h   (stride 1, KW = 3, 64 output channels, padded width <= 128)
    (2, 8, 8, 64, 3, 1, 1),
    (8, 56, 56, 64, 3, 1, 1),
    (2, 12, 12, 64, 3, 0, 1),
    (3, 13, 9, 128, 2, 1, 2),
    (2, 57, 31, 64, 1, 1, 1),
    (2, 126, 5, 64, 3, 1, 1),
    (2, 20, 100, 64, 3, 1, 1),
    (1, 40, 126, 64, 3, 1, 1),    # one padded row fills the 128 MMA rows
    (5, 28, 28, 128, 1, 1, 1),
    (1, 3, 3, 64, 3, 1, 1),
    (3, 9, 30, 64, 3, 1, 1),      # four padded rows per tile: warps start mid-row
    (2, 17, 62, 128, 2, 2, 1),    # two-pixel padding: the padded row is wider than the output row by more than the shift
]


@pytest.fixture(autouse=True)
def _status_clean(hb_lib):
    yield
    from heron_b200 import _lib
    assert _lib.last_status() == 0, "a bounded device-side wait ran out"


@pytest.mark.parametrize("case", FUSED_CASES)
def test_fused_row_strip_conv_fp16(K, co, case):
    N, H, W, CI, KH, p, dh = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, H, W, CI)).astype(np.float16)
    w = (rng.standard_normal((KH, 3, CI, 64)) / np.sqrt(KH * 3 * CI)).astype(np.float16)
    for od in (np.float32, np.float16):
        want = co.conv2d_nhwc_f16(x, w, 1, p, (dh, 1), od)
        got = k_conv(K, x, w, 1, p, (dh, 1), out_dtype=od, knobs=dict(conv_algo=4))
        check(got, want, "fused-row strip %s" % (case,))


from hypothesis import HealthCheck, given, settings, strategies as st


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck))
@given(N=st.integers(1, 3), H=st.integers(1, 40), W=st.integers(1, 120), CI=st.sampled_from([64, 128]),
       KH=st.integers(1, 3), pad=st.integers(0, 2), dh=st.integers(1, 2), half_out=st.booleans(),
       max_ctas=st.sampled_from([0, 1, 3]), seed=st.integers(0, 2 ** 20))
def test_fused_row_strip_random_geometry(K, co, N, H, W, CI, KH, pad, dh, half_out, max_ctas, seed):
    """Random stride-1 geometries: tiles of one to many padded rows, a last tile that hangs over the
    image, one-row images, dilation along H, few CTAs (ring, accumulators and the exchange's two
    buffers reused many times)."""
    from heron_b200._lib import HB_ERR_KNOB, HeronB200Error
    if H + 2 * pad < (KH - 1) * dh + 1 or W + 2 * pad < 3:
        return
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, H, W, CI)).astype(np.float16)
    w = (rng.standard_normal((KH, 3, CI, 64)) / np.sqrt(KH * 3 * CI)).astype(np.float16)
    od = np.float16 if half_out else np.float32
    # the constraint model's own rule (the padded row within the 128 MMA rows; filter, two strips
    # and the exchange within shared memory) says which geometries the library takes
    from heron_b200.schedule.context.context import B200_LIMITS
    from heron_b200.schedule.sched_op import strip_fused_applies
    geom = dict(stride=(1, 1), dilation=(dh, 1), CI=CI, CO=64, KH=KH, KW=3, padding=pad, H=H, W=W, in_dtype="float16")
    feasible = strip_fused_applies(geom, 2, 2 if half_out else 4, B200_LIMITS)
    try:
        got = k_conv(K, x, w, 1, pad, (dh, 1), out_dtype=od, knobs=dict(conv_algo=4, max_ctas=max_ctas))
    except HeronB200Error as e:
        assert e.status == HB_ERR_KNOB and not feasible
        return
    assert feasible
    check(got, co.conv2d_nhwc_f16(x, w, 1, pad, (dh, 1), od), "fused-row strip %s" % ((N, H, W, CI, KH, pad, dh),))


def test_fused_row_strip_one_hot_channels(K, co):
    """Every (tap, input channel) lands on its own output pixel and channel: a filter that is
    one-hot per tap maps input channel c of the tap's pixel to output channel (c * 7 + tap) % 64,
    so a column group added at the wrong shift, or a boundary lane fed from the wrong exchange
    row, changes exact small integers."""
    rng = np.random.default_rng(3)
    x = rng.integers(-4, 5, (2, 9, 43, 64)).astype(np.float16)
    w = np.zeros((3, 3, 64, 64), np.float16)
    for tap in range(9):
        for c in range(64):
            w[tap // 3, tap % 3, c, (c * 7 + tap) % 64] = 1.0
    got = k_conv(K, x, w, 1, 1, 1, out_dtype=np.float32, knobs=dict(conv_algo=4)).cpu().numpy()
    assert np.array_equal(got, co.conv2d_nhwc_f16(x, w, 1, 1, 1, np.float32))  # small integers: exact


def test_fused_row_strip_walks_its_ring_and_relaunches(K, co):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((6, 30, 30, 64)).astype(np.float16)
    w = (rng.standard_normal((3, 3, 64, 64)) / 24.0).astype(np.float16)
    out = poison((6, 30, 30, 64), torch.float16)
    plan = K.plan_conv2d_nhwc(dev(x), dev(w), stride=1, padding=1, dilation=1, out=out,
                              knobs=dict(conv_algo=4, max_ctas=1))
    kn = plan.knobs()
    assert kn["conv_algo"] == 4 and kn["grid"] == 1 and kn["tile_n"] == 192, kn
    plan.launch()
    check(out, co.conv2d_nhwc_f16(x, w, 1, 1, 1, np.float16), "fused-row strip, one CTA")
    first = out.clone()
    out.view(torch.uint8).fill_(0xCD)
    plan.launch()
    assert torch.equal(out, first)


def test_fused_row_strip_refused_where_it_does_not_apply(K):
    from heron_b200._lib import HB_ERR_KNOB, HeronB200Error
    x = torch.zeros(2, 14, 14, 64, dtype=torch.float16, device="cuda")
    cases = [
        (torch.zeros(3, 3, 64, 128, dtype=torch.float16, device="cuda"), 1, 1, 1),   # 128 output channels
        (torch.zeros(3, 2, 64, 64, dtype=torch.float16, device="cuda"), 1, 1, 1),    # KW = 2
        (torch.zeros(3, 3, 64, 64, dtype=torch.float16, device="cuda"), 2, 1, 1),    # stride 2
        (torch.zeros(3, 3, 64, 64, dtype=torch.float16, device="cuda"), 1, 2, 2),    # dilation along W
    ]
    for w, s, p, d in cases:
        with pytest.raises(HeronB200Error) as e:
            K.conv2d_nhwc(x, w, s, p, d, knobs=dict(conv_algo=4))
        assert e.value.status == HB_ERR_KNOB
    xi = torch.zeros(2, 14, 14, 128, dtype=torch.uint8, device="cuda")
    wi = torch.zeros(3, 3, 128, 128, dtype=torch.int8, device="cuda")
    with pytest.raises(HeronB200Error) as e:
        K.conv2d_nhwc(xi, wi, 1, 1, 1, knobs=dict(conv_algo=4))  # integer operands
    assert e.value.status == HB_ERR_KNOB


def test_cfg3_full_size_on_the_fused_row_strip_kernel(K, co):
    from heron_b200.workloads import make_inputs
    x, w = make_inputs("cfg3_conv_f16_resnet_s2")
    out = k_conv(K, x, w, 1, 1, 1, out_dtype=np.float16, knobs=dict(conv_algo=4))
    for n in (0, 13, 31):
        check(out[n:n + 1], co.conv2d_nhwc_f16(x[n:n + 1], w, 1, 1, 1, np.float16), "cfg3 image %d" % n)


@pytest.mark.parametrize("args", [
    [16, 20, 20, 64, 64, 3, 3, 1, 1, 1, "float16", "float16"],
    [16, 12, 70, 64, 64, 3, 3, 1, 1, 1, "float16", "float32"],
])
def test_knob_space_reaches_every_conv_algorithm(K, co, args):
    """Random feasible points of the operator's knob space (the constraint model's conv-algorithm
    rule lists the fused-row form where the library accepts it): every point runs and matches the
    oracle, and the sweep meets the fused-row form and at least two of the others."""
    import random
    from heron_b200.ops import cuda as heron_cuda
    from test_gpu_parity import _task
    t = _task(heron_cuda, "c2d_nhwc", args, "GPU_TENSOR_CORE")
    N, H, W, CI, CO = args[:5]
    rng = np.random.default_rng(H)
    x = rng.standard_normal((N, H, W, CI)).astype(np.float16)
    w = (rng.standard_normal((3, 3, CI, CO)) / np.sqrt(9 * CI)).astype(np.float16)
    od = np.float16 if args[-1] == "float16" else np.float32
    want = co.conv2d_nhwc_f16(x, w, 1, 1, 1, od)
    tin = [dev(x), dev(w)]
    random.seed(23)
    seen, algos = set(), set()
    for _ in range(150):
        if len(seen) >= 40:
            break
        t.knob_manager.randSample()
        handle, targs = t.instantiate(t.knob_manager)
        key = tuple(sorted(handle.knobs.items()))
        if key in seen:
            continue
        seen.add(key)
        algos.add(handle.knobs.get("conv_algo"))
        out = poison(targs[-1].shape, torch.float16 if od == np.float16 else torch.float32)
        handle(*tin, out)
        check(out, want, str(handle.knobs))
    assert 4 in algos and len(algos) >= 3, algos


@pytest.mark.parametrize("case", [(2, 64, 14, 14), (3, 64, 30, 41), (2, 64, 9, 100), (16, 64, 56, 56)])
def test_fused_row_strip_channel_major_output(K, co, case):
    """The NCHW operator on the fused-row form: the epilogue's channel-major stores (no staging
    tile, each lane writes its pixel's channels plane by plane), fp16 and fp32 outputs."""
    N, CI, H, W = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, CI, H, W)).astype(np.float16)
    w = (rng.standard_normal((64, CI, 3, 3)) / np.sqrt(9 * CI)).astype(np.float16)
    for od, td in ((np.float16, torch.float16), (np.float32, torch.float32)):
        out = poison((N, 64, H, W), td)
        plan = K.plan_conv2d_nchw(dev(x), dev(w), stride=1, padding=1, out=out, knobs=dict(conv_algo=4))
        assert plan.knobs()["conv_algo"] == 4
        plan.launch()
        check(out, co.conv2d_nchw(x, w, 1, 1, od), "fused-row strip, NCHW %s" % (case,))
