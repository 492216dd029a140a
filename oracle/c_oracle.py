"""ctypes front end of heron_oracle.c (numpy arrays in, numpy arrays out).  TEST INFRASTRUCTURE ONLY."""
import ctypes

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        _build.build()  # no-op unless the source is newer than the library
        _lib = ctypes.CDLL(_build.ORACLE_SO)
        _lib.oracle_half_to_float.restype = ctypes.c_float
        _lib.oracle_half_to_float.argtypes = [ctypes.c_uint16]
        _lib.oracle_float_to_half.restype = ctypes.c_uint16
        _lib.oracle_float_to_half.argtypes = [ctypes.c_float]
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _signed(a):
    if a.dtype == np.int8:
        return 1
    if a.dtype == np.uint8:
        return 0
    raise TypeError("expected uint8 / int8, got %s" % a.dtype)


def _c(a):
    return np.ascontiguousarray(a)


def gemm_int(a, b):
    a, b = _c(a), _c(b)
    M, K = a.shape
    N = b.shape[0]
    out = np.empty((M, N), dtype=np.int32)
    lib().oracle_gemm_i8(_p(a), _p(b), _p(out), M, K, N, _signed(a), _signed(b))
    return out


def bmm_int(a, b):
    a, b = _c(a), _c(b)
    B, M, K = a.shape
    N = b.shape[1]
    out = np.empty((B, M, N), dtype=np.int32)
    lib().oracle_bmm_i8(_p(a), _p(b), _p(out), B, M, K, N, _signed(a), _signed(b))
    return out


def gemm_f16(a, b):
    a, b = _c(a), _c(b)
    assert a.dtype == np.float16 and b.dtype == np.float16
    M, K = a.shape
    N = b.shape[0]
    out = np.empty((M, N), dtype=np.float32)
    lib().oracle_gemm_f16(_p(a), _p(b), _p(out), M, K, N)
    return out


def bmm_f16(a, b):
    a, b = _c(a), _c(b)
    B, M, K = a.shape
    N = b.shape[1]
    out = np.empty((B, M, N), dtype=np.float32)
    lib().oracle_bmm_f16(_p(a), _p(b), _p(out), B, M, K, N)
    return out


def _pair(v):
    return (v, v) if isinstance(v, int) else (int(v[0]), int(v[1]))


def _out_hw(H, W, KH, KW, stride, pad, dilation):
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    L = lib()
    return (L.oracle_conv_out_extent(H, KH, sh, pad, dh), L.oracle_conv_out_extent(W, KW, sw, pad, dw))


def conv2d_nhwc_int(x, w, stride=1, pad=0, dilation=1):
    x, w = _c(x), _c(w)
    N, H, W, CI = x.shape
    KH, KW, _, CO = w.shape
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    HO, WO = _out_hw(H, W, KH, KW, stride, pad, dilation)
    out = np.empty((N, HO, WO, CO), dtype=np.int32)
    lib().oracle_conv2d_nhwc_i8(_p(x), _p(w), _p(out), N, H, W, CI, CO, KH, KW, sh, sw, pad, dh, dw,
                                _signed(x), _signed(w))
    return out


def conv2d_nhwc_f16(x, w, stride=1, pad=0, dilation=1, out_dtype=np.float32):
    x, w = _c(x), _c(w)
    assert x.dtype == np.float16 and w.dtype == np.float16
    N, H, W, CI = x.shape
    KH, KW, _, CO = w.shape
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    HO, WO = _out_hw(H, W, KH, KW, stride, pad, dilation)
    half = np.dtype(out_dtype) == np.float16
    out = np.empty((N, HO, WO, CO), dtype=np.float16 if half else np.float32)
    lib().oracle_conv2d_nhwc_f16(_p(x), _p(w), _p(out), N, H, W, CI, CO, KH, KW, sh, sw, pad, dh, dw,
                                 1 if half else 0)
    return out


def conv2d_nhwc_packed(x, w_packed, stride=1, pad=0, dilation=1):
    x, w_packed = _c(x), _c(w_packed)
    assert x.dtype == np.uint8 and w_packed.dtype == np.int8
    N, H, W, CI = x.shape
    OC, KH, KW, IC, sco, sci = w_packed.shape
    assert sci == 4 and IC * 4 == CI
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    HO, WO = _out_hw(H, W, KH, KW, stride, pad, dilation)
    out = np.empty((N, HO, WO, OC, sco), dtype=np.int32)
    lib().oracle_conv2d_nhwc_packed(_p(x), _p(w_packed), _p(out), N, H, W, CI, OC * sco, KH, KW, sh,
                                    sw, pad, dh, dw, sco)
    return out


def conv2d_nchw(x, w, stride=1, pad=0, out_dtype=None):
    """NCHW input, OIHW filter; integer operands give int32, fp16 operands float32 (or fp16)."""
    x, w = _c(x), _c(w)
    N, CI, H, W = x.shape
    CO, _, KH, KW = w.shape
    sh, sw = _pair(stride)
    HO, WO = _out_hw(H, W, KH, KW, stride, pad, 1)
    if x.dtype == np.float16:
        half = out_dtype is not None and np.dtype(out_dtype) == np.float16
        out = np.empty((N, CO, HO, WO), dtype=np.float16 if half else np.float32)
        lib().oracle_conv2d_nchw(_p(x), _p(w), _p(out), N, H, W, CI, CO, KH, KW, sh, sw, pad, 2 if half else 1, 0, 0)
    else:
        out = np.empty((N, CO, HO, WO), dtype=np.int32)
        lib().oracle_conv2d_nchw(_p(x), _p(w), _p(out), N, H, W, CI, CO, KH, KW, sh, sw, pad, 0, _signed(x),
                                 _signed(w))
    return out


def gemv(a, x, out_dtype=None):
    """The tensor-core gemv: a (M,K), x (1,K) -> (M,8) with the product in column 0."""
    a, x = _c(a), _c(x)
    M, K = a.shape
    assert x.shape == (1, K)
    if a.dtype == np.float16:
        half = out_dtype is not None and np.dtype(out_dtype) == np.float16
        out = np.empty((M, 8), dtype=np.float16 if half else np.float32)
        lib().oracle_gemv(_p(a), _p(x), _p(out), M, K, 2 if half else 1, 0, 0)
    else:
        out = np.empty((M, 8), dtype=np.int32)
        lib().oracle_gemv(_p(a), _p(x), _p(out), M, K, 0, _signed(a), _signed(x))
    return out


def conv1d_ncw(x, w, stride=1, pad=0, out_dtype=None):
    x, w = _c(x), _c(w)
    N, CI, W = x.shape
    CO, _, KW = w.shape
    WO = (W - KW + 2 * pad) // stride + 1
    if x.dtype == np.float16:
        half = out_dtype is not None and np.dtype(out_dtype) == np.float16
        out = np.empty((N, CO, WO), dtype=np.float16 if half else np.float32)
        lib().oracle_conv1d_ncw(_p(x), _p(w), _p(out), N, W, CI, CO, KW, stride, pad, 2 if half else 1, 0, 0)
    else:
        out = np.empty((N, CO, WO), dtype=np.int32)
        lib().oracle_conv1d_ncw(_p(x), _p(w), _p(out), N, W, CI, CO, KW, stride, pad, 0, _signed(x), _signed(w))
    return out


def conv1d_nwc_packed(x, w_packed, stride=1, pad=0, dilation=1):
    x, w_packed = _c(x), _c(w_packed)
    assert x.dtype == np.uint8 and w_packed.dtype == np.int8
    N, W, CI = x.shape
    OC, KW, IC, sco, sci = w_packed.shape
    assert sci == 4 and IC * 4 == CI
    WO = (W - ((KW - 1) * dilation + 1) + 2 * pad) // stride + 1
    out = np.empty((N, WO, OC, sco), dtype=np.int32)
    lib().oracle_conv1d_nwc_packed(_p(x), _p(w_packed), _p(out), N, W, CI, OC * sco, KW, stride, pad,
                                   dilation, sco)
    return out


def scan(a, N, out_dtype=None):
    a = _c(a)
    M, K = a.shape
    if a.dtype == np.float16:
        half = out_dtype is not None and np.dtype(out_dtype) == np.float16
        out = np.empty((M, N), dtype=np.float16 if half else np.float32)
        lib().oracle_scan(_p(a), _p(out), M, N, K, 2 if half else 1, 0)
    else:
        out = np.empty((M, N), dtype=np.int32)
        lib().oracle_scan(_p(a), _p(out), M, N, K, 0, _signed(a))
    return out


def conv3d_ncdhw(x, w, stride=1, pad=0, out_dtype=None):
    x, w = _c(x), _c(w)
    N, CI, D, H, W = x.shape
    CO, _, KD, KH, KW = w.shape
    sd, sh, sw = (stride, stride, stride) if isinstance(stride, int) else tuple(int(v) for v in stride)
    shape = (N, CO, (D - KD + 2 * pad) // sd + 1, (H - KH + 2 * pad) // sh + 1, (W - KW + 2 * pad) // sw + 1)
    if x.dtype == np.float16:
        half = out_dtype is not None and np.dtype(out_dtype) == np.float16
        out = np.empty(shape, dtype=np.float16 if half else np.float32)
        lib().oracle_conv3d_ncdhw(_p(x), _p(w), _p(out), N, D, H, W, CI, CO, KD, KH, KW, sd, sh, sw, pad,
                                  2 if half else 1, 0, 0)
    else:
        out = np.empty(shape, dtype=np.int32)
        lib().oracle_conv3d_ncdhw(_p(x), _p(w), _p(out), N, D, H, W, CI, CO, KD, KH, KW, sd, sh, sw, pad, 0,
                                  _signed(x), _signed(w))
    return out
