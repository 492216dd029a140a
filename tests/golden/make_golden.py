"""Generates tests/golden/kat.npz: small known-answer cases for the operators on the hot path.

    python tests/golden/make_golden.py

The reference has no golden tensor values for these operators (it never checks results) and
cannot run here (it needs Apache TVM), so these vectors do NOT come from the reference: the
hand-checkable cases are written down from the operator definitions
(ops/cuda/dense.py:12-17, ops/cuda/batch_matmul.py:14-19, ops/cuda/conv2d.py:168-196,
ops/x86/conv2d_int8.py:74-93) and the seeded cases are outputs of the numpy restatement
(oracle/np_oracle.py) frozen at the time of writing, so that a later change to either oracle or
to the kernels shows up as a diff against committed bytes.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import np_oracle as npo  # noqa: E402


def build_cases():
    cases = {}
    rng = np.random.Generator(np.random.PCG64(777))

    # -- hand-checkable ---------------------------------------------------------------------
    # identity B: C == A (B is (N,K), so B = I gives C[i,j] = A[i,j])
    a = rng.integers(0, 256, size=(16, 16), dtype=np.uint8)
    eye = np.eye(16, dtype=np.int8)
    cases["gemm_u8s8_identity"] = dict(a=a, b=eye, out=a.astype(np.int32))
    # extremes: 255 * -128 summed 64 times
    a = np.full((8, 64), 255, dtype=np.uint8)
    b = np.full((16, 64), -128, dtype=np.int8)
    cases["gemm_u8s8_extremes"] = dict(a=a, b=b, out=np.full((8, 16), 64 * 255 * -128, dtype=np.int32))
    # s8 x s8 extremes: (-128)*(-128)*K and (-128)*127*K
    a = np.full((4, 32), -128, dtype=np.int8)
    b = np.stack([np.full(32, -128, dtype=np.int8), np.full(32, 127, dtype=np.int8)] * 8)
    out = np.tile(np.array([32 * 16384, 32 * -16256], dtype=np.int32), (4, 8))
    cases["gemm_s8s8_extremes"] = dict(a=a, b=b, out=out)
    # one-hot rows: row i of A selects column k=i of B^T -> C[i,j] = B[j,i]
    a = np.eye(8, 16, dtype=np.float16)
    b = rng.standard_normal((16, 16)).astype(np.float16)
    cases["gemm_f16_onehot"] = dict(a=a, b=b, out=b[:, :8].T.astype(np.float32))
    # conv with a centre-only 3x3 filter of identity channels: out == in
    x = rng.integers(0, 256, size=(1, 5, 5, 32), dtype=np.uint8)
    w = np.zeros((3, 3, 32, 32), dtype=np.int8)
    w[1, 1] = np.eye(32, dtype=np.int8)
    cases["conv_u8s8_centre_identity"] = dict(x=x, w=w, stride=1, pad=1, dil=1, out=x.astype(np.int32))
    # all-ones: each output counts the taps that fall inside the image
    x = np.ones((1, 4, 4, 32), dtype=np.uint8)
    w = np.ones((3, 3, 32, 32), dtype=np.int8)
    cnt = np.array([[4, 6, 6, 4], [6, 9, 9, 6], [6, 9, 9, 6], [4, 6, 6, 4]], dtype=np.int32) * 32
    cases["conv_u8s8_ones_padding"] = dict(x=x, w=w, stride=1, pad=1, dil=1,
                                           out=np.broadcast_to(cnt[None, :, :, None], (1, 4, 4, 32)).copy())

    # -- seeded, frozen outputs of the numpy restatement ----------------------------------------
    a = rng.integers(0, 256, size=(64, 64), dtype=np.uint8)
    b = rng.integers(-128, 128, size=(64, 64)).astype(np.int8)
    cases["gemm_u8s8_64"] = dict(a=a, b=b, out=npo.gemm_int(a, b))
    a = rng.integers(-128, 128, size=(3, 40, 48)).astype(np.int8)
    b = rng.integers(-128, 128, size=(3, 24, 48)).astype(np.int8)
    cases["bmm_s8s8_ragged"] = dict(a=a, b=b, out=npo.bmm_int(a, b))
    a = (rng.standard_normal((48, 72)) / np.sqrt(72)).astype(np.float16)
    b = rng.standard_normal((40, 72)).astype(np.float16)
    cases["gemm_f16_48x40x72"] = dict(a=a, b=b, out=npo.gemm_f16(a, b))
    x = rng.integers(0, 256, size=(2, 7, 7, 32), dtype=np.uint8)
    w = rng.integers(-128, 128, size=(3, 3, 32, 32)).astype(np.int8)
    cases["conv_u8s8_7x7"] = dict(x=x, w=w, stride=1, pad=1, dil=1, out=npo.conv2d_nhwc_int(x, w, 1, 1, 1))
    cases["conv_u8s8_7x7_s2"] = dict(x=x, w=w, stride=2, pad=1, dil=1, out=npo.conv2d_nhwc_int(x, w, 2, 1, 1))
    cases["conv_u8s8_7x7_d2"] = dict(x=x, w=w, stride=1, pad=2, dil=2, out=npo.conv2d_nhwc_int(x, w, 1, 2, 2))
    xf = rng.standard_normal((2, 6, 6, 16)).astype(np.float16)
    wf = (rng.standard_normal((3, 3, 16, 32)) / 12.0).astype(np.float16)
    cases["conv_f16_6x6"] = dict(x=xf, w=wf, stride=1, pad=1, dil=1, out=npo.conv2d_nhwc_f16(xf, wf, 1, 1, 1))
    cases["conv_f16_6x6_halfout"] = dict(x=xf, w=wf, stride=1, pad=1, dil=1,
                                         out=npo.conv2d_nhwc_f16(xf, wf, 1, 1, 1, np.float16))
    wp = npo.pack_filter_x86(w, 32)
    cases["conv_packed_OhwI32o4i"] = dict(x=x, w=wp, stride=1, pad=1, dil=1,
                                          out=npo.conv2d_nhwc_packed(x, wp, 1, 1, 1))
    return cases


def build_neighbour_cases():
    """kat_neighbours.npz: gemv (ops/cuda/gemv.py:12-30) and the 1-D convolutions
    (ops/cuda/conv1d.py:23-69, ops/x86/conv1d_int8.py:53-84), same two kinds of case."""
    cases = {}
    rng = np.random.Generator(np.random.PCG64(778))
    # gemv, one-hot rows of A: out[i,0] = x[i], columns 1..7 zero
    a = np.eye(16, 32, dtype=np.uint8)
    x = rng.integers(-128, 128, size=(1, 32)).astype(np.int8)
    out = np.zeros((16, 8), dtype=np.int32)
    out[:, 0] = x[0, :16]
    cases["gemv_u8s8_onehot"] = dict(a=a, x=x, out=out)
    a = (rng.standard_normal((40, 48)) / 7.0).astype(np.float16)
    x = rng.standard_normal((1, 48)).astype(np.float16)
    cases["gemv_f16_40x48"] = dict(a=a, x=x, out=npo.gemv(a, x))
    # conv1d NCW, all ones, KW = 3, pad 4 (wider than the filter, as in the reference's own cases):
    # output position q sees the taps q-4 .. q-2 of a width-6 input
    xi = np.ones((1, 16, 6), dtype=np.uint8)
    wi = np.ones((32, 16, 3), dtype=np.int8)
    taps = np.array([0, 0, 1, 2, 3, 3, 3, 3, 2, 1, 0, 0], dtype=np.int32) * 16
    cases["c1d_ncw_ones_wide_padding"] = dict(x=xi, w=wi, stride=1, pad=4,
                                              out=np.broadcast_to(taps[None, None, :], (1, 32, 12)).copy())
    xf = rng.standard_normal((2, 16, 21)).astype(np.float16)
    wf = (rng.standard_normal((24, 16, 3)) / 7.0).astype(np.float16)
    cases["c1d_ncw_f16_s2"] = dict(x=xf, w=wf, stride=2, pad=1, out=npo.conv1d_ncw(xf, wf, 2, 1))
    # conv1d NWC packed, one tap of identity channels: out == in
    xi = rng.integers(0, 256, size=(2, 9, 32), dtype=np.uint8)
    w = np.eye(32, dtype=np.int8)[None]
    cases["c1d_nwc_packed_identity"] = dict(x=xi, w=npo.pack_filter_x86_1d(w, 32), stride=1, pad=0, dil=1,
                                            out=xi.astype(np.int32).reshape(2, 9, 1, 32))
    xi = rng.integers(0, 256, size=(2, 23, 32), dtype=np.uint8)
    w = rng.integers(-128, 128, size=(3, 32, 64)).astype(np.int8)
    wp = npo.pack_filter_x86_1d(w, 64)
    cases["c1d_nwc_packed_d2"] = dict(x=xi, w=wp, stride=1, pad=4, dil=2,
                                      out=npo.conv1d_nwc_packed(xi, wp, 1, 4, 2))
    return cases


def _write(name, cases):
    flat = {}
    for cname, case in cases.items():
        for key, val in case.items():
            flat["%s/%s" % (cname, key)] = np.asarray(val)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), name)
    np.savez_compressed(path, **flat)
    print("wrote", path, os.path.getsize(path), "bytes,", len(cases), "cases")


def main():
    _write("kat.npz", build_cases())
    _write("kat_neighbours.npz", build_neighbour_cases())


if __name__ == "__main__":
    main()
