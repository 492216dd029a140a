"""hb_conv2d_nhwc_packed_noalloc: the packed-filter conv for hosts that cannot give the library a
workspace and may not allocate one — the reference's calling convention passes a built operator
its tensors and nothing else, and cudaMalloc is off limits inside a timed loop or a stream capture.

The entry point unpacks the filter into a 4 MiB array that is part of the library image, so it
must give exactly what hb_conv2d_nhwc_packed gives with a caller-owned buffer.  Two calls in a
row with different filters check that the shared array carries nothing over from one call to the
next.  The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import np_oracle as npo

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _both(lib, x, wp, CO, KH, KW, stride, pad, dil, sco):
    """Runs the caller-scratch entry point and the no-allocation one on the same inputs."""
    N, H, W, CI = x.shape
    HO = (H - ((KH - 1) * dil + 1) + 2 * pad) // stride + 1
    WO = (W - ((KW - 1) * dil + 1) + 2 * pad) // stride + 1
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    want = torch.full((N, HO, WO, CO // sco, sco), -1, dtype=torch.int32, device="cuda")
    scratch = torch.empty(lib.hb_conv2d_packed_scratch_bytes(CI, CO, KH, KW), dtype=torch.int8, device="cuda")
    rc = lib.hb_conv2d_nhwc_packed(_ptr(x), _ptr(wp), _ptr(want), N, H, W, CI, CO, KH, KW, stride, stride, pad,
                                   dil, dil, sco, _ptr(scratch), scratch.numel(), None, stream)
    assert rc == 0
    got = torch.full_like(want, -2)
    rc = lib.hb_conv2d_nhwc_packed_noalloc(_ptr(x), _ptr(wp), _ptr(got), N, H, W, CI, CO, KH, KW, stride, stride,
                                           pad, dil, dil, sco, None, stream)
    assert rc == 0
    torch.cuda.synchronize()
    return got, want


def test_noalloc_matches_caller_scratch_twice_in_a_row(hb_lib):
    from heron_b200 import _lib
    assert torch.cuda.is_available()
    assert hb_lib.hb_conv2d_packed_noalloc_max_bytes() == 4 << 20
    rng = np.random.default_rng(99)

    # first call: 3x3, 64 -> 128 channels, sco 64
    x1 = rng.integers(0, 256, (4, 9, 9, 64), dtype=np.uint8)
    w1 = rng.integers(-128, 128, (3, 3, 64, 128)).astype(np.int8)
    wp1 = npo.pack_filter_x86(w1, 64)
    got, want = _both(hb_lib, torch.from_numpy(x1).cuda(), torch.from_numpy(wp1).cuda(), 128, 3, 3, 1, 1, 1, 64)
    assert torch.equal(got, want)
    assert np.array_equal(got.cpu().numpy(), npo.conv2d_nhwc_packed(x1, wp1, 1, 1, 1))

    # second call right after, smaller and different filter: only its own bytes may be used
    x2 = rng.integers(0, 256, (2, 7, 7, 32), dtype=np.uint8)
    w2 = rng.integers(-128, 128, (1, 1, 32, 96)).astype(np.int8)
    wp2 = npo.pack_filter_x86(w2, 32)
    got, want = _both(hb_lib, torch.from_numpy(x2).cuda(), torch.from_numpy(wp2).cuda(), 96, 1, 1, 2, 0, 1, 32)
    assert torch.equal(got, want)
    assert np.array_equal(got.cpu().numpy(), npo.conv2d_nhwc_packed(x2, wp2, 2, 0, 1))
    assert _lib.last_status() == 0


def test_noalloc_refuses_filters_beyond_its_array(hb_lib):
    from heron_b200 import _lib
    # 3*3*1024*1024 bytes = 9 MiB > 4 MiB: refused before anything is launched
    x = torch.zeros(1, 4, 4, 1024, dtype=torch.uint8, device="cuda")
    wp = torch.zeros(16, 3, 3, 256, 64, 4, dtype=torch.int8, device="cuda")
    out = torch.zeros(1, 4, 4, 16, 64, dtype=torch.int32, device="cuda")
    rc = hb_lib.hb_conv2d_nhwc_packed_noalloc(_ptr(x), _ptr(wp), _ptr(out), 1, 4, 4, 1024, 1024, 3, 3, 1, 1, 1, 1, 1,
                                              64, None, None)
    assert rc == _lib.HB_ERR_STATIC_SCRATCH
    assert "4 MiB" in _lib.status_string(rc)
