"""ctypes front end of dlboost_baseline.c — the timed CPU baseline.  TEST / BENCHMARK INFRASTRUCTURE ONLY."""
import ctypes
import os

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_build.DLBOOST_SO):
            _build.build()
        _lib = ctypes.CDLL(_build.DLBOOST_SO)
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def has_vnni():
    return bool(lib().dlb_has_vnni())


def has_avx512():
    return bool(lib().dlb_has_avx512())


def max_threads():
    return int(lib().dlb_max_threads())


def set_threads(n):
    lib().dlb_set_threads(int(n))


class GemmU8S8:
    """u8 (M,K) x s8 (N,K) -> s32, scratch allocated once so that repeated calls time the kernel."""

    def __init__(self, M, K, N):
        self.shape = (M, K, N)
        self.pack = np.empty(N * K, dtype=np.int8)
        self.out = np.empty((M, N), dtype=np.int32)

    def __call__(self, a, b):
        M, K, N = self.shape
        lib().dlb_gemm_u8s8(_p(a), _p(b), _p(self.out), M, K, N, _p(self.pack))
        return self.out


class BmmS8S8:
    def __init__(self, B, M, K, N):
        self.shape = (B, M, K, N)
        self.a_bias = np.empty(B * M * K, dtype=np.uint8)
        self.pack = np.empty(N * K, dtype=np.int8)
        self.colsum = np.empty(N, dtype=np.int32)
        self.out = np.empty((B, M, N), dtype=np.int32)

    def __call__(self, a, b):
        B, M, K, N = self.shape
        lib().dlb_bmm_s8s8(_p(a), _p(b), _p(self.out), B, M, K, N, _p(self.a_bias), _p(self.pack),
                           _p(self.colsum))
        return self.out


class BmmU8S8:
    def __init__(self, B, M, K, N):
        self.shape = (B, M, K, N)
        self.pack = np.empty(N * K, dtype=np.int8)
        self.out = np.empty((B, M, N), dtype=np.int32)

    def __call__(self, a, b):
        B, M, K, N = self.shape
        lib().dlb_bmm_u8s8(_p(a), _p(b), _p(self.out), B, M, K, N, _p(self.pack))
        return self.out


class ConvPacked:
    """u8 NHWC x packed s8 filter (CO/sco,KH,KW,CI/4,sco,4) -> s32 (N,HO,WO,CO/sco,sco)."""

    def __init__(self, N, H, W, CI, CO, KH, KW, stride, pad, dilation, sco=64):
        sh, sw = (stride, stride) if isinstance(stride, int) else stride
        dh, dw = (dilation, dilation) if isinstance(dilation, int) else dilation
        self.args = (N, H, W, CI, CO, KH, KW, sh, sw, pad, dh, dw, sco)
        HO = (H - ((KH - 1) * dh + 1) + 2 * pad) // sh + 1
        WO = (W - ((KW - 1) * dw + 1) + 2 * pad) // sw + 1
        self.out = np.empty((N, HO, WO, CO // sco, sco), dtype=np.int32)

    def __call__(self, x, w_packed):
        lib().dlb_conv2d_nhwc_packed(_p(x), _p(w_packed), _p(self.out), *self.args)
        return self.out


class GemmF16:
    """fp16 (M,K) x fp16 (N,K) -> fp32 through an fp32 AVX512 loop (the fp16 configs' CPU column)."""

    def __init__(self, M, K, N):
        self.shape = (M, K, N)
        self.a32 = np.empty(M * K, dtype=np.float32)
        self.b32 = np.empty(N * K, dtype=np.float32)
        self.out = np.empty((M, N), dtype=np.float32)

    def __call__(self, a, b):
        M, K, N = self.shape
        lib().dlb_gemm_f16(_p(a), _p(b), _p(self.out), M, K, N, _p(self.a32), _p(self.b32))
        return self.out
