"""numpy restatement of the reference's operator math.  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED: the reference ships no golden tensor values for these operators and cannot run
in this environment (it needs Apache TVM, un-vendored and un-pinned); what this file follows is
the arithmetic of the reference's ``te.compute`` bodies, cited per function.  It exists beside the
C restatement (heron_oracle.c) so that the two, written independently in different styles
(vectorised matmul / explicit im2col here, scalar loops there), can be checked against each other.

Integer results are exact int32 (computed in int64, checked to fit); fp16 inputs are widened to
float64 and accumulated there.
"""
import numpy as np


def _as_i64(x):
    if x.dtype not in (np.uint8, np.int8):
        raise TypeError("integer oracle takes uint8 / int8 operands, got %s" % x.dtype)
    return x.astype(np.int64)


def _to_i32(acc):
    if acc.size and (acc.max() > np.iinfo(np.int32).max or acc.min() < np.iinfo(np.int32).min):
        raise OverflowError("sum leaves int32: the reference's int32 accumulation would wrap")
    return acc.astype(np.int32)


def gemm_int(a, b):
    """out[i,j] = sum_k int32(a[i,k]) * int32(b[j,k]); ops/x86/dense.py:14-18, ops/cuda/dense.py:12-17."""
    return _to_i32(_as_i64(a) @ _as_i64(b).T)


def bmm_int(a, b):
    """out[n,i,j] = sum_k a[n,i,k] * b[n,j,k]; ops/x86/batch_matmul.py:15-20."""
    return _to_i32(np.einsum("bik,bjk->bij", _as_i64(a), _as_i64(b)))


def gemm_f16(a, b):
    """fp16 operands (B is (N,K)), float64 accumulation, float32 result; ops/cuda/dense.py:12-17."""
    assert a.dtype == np.float16 and b.dtype == np.float16
    return (a.astype(np.float64) @ b.astype(np.float64).T).astype(np.float32)


def bmm_f16(a, b):
    """ops/cuda/batch_matmul.py:14-19 with fp16 operands."""
    assert a.dtype == np.float16 and b.dtype == np.float16
    return np.einsum("bik,bjk->bij", a.astype(np.float64), b.astype(np.float64)).astype(np.float32)


def _pair(v):
    return (v, v) if isinstance(v, int) else (int(v[0]), int(v[1]))


def conv_out_extent(size, k, stride, pad, dil):
    """(size - dilated_k + 2*pad) // stride + 1; ops/cuda/conv2d.py:165-175."""
    return (size - ((k - 1) * dil + 1) + 2 * pad) // stride + 1


def _im2col(x, KH, KW, stride, pad, dilation):
    """(N,H,W,C) -> (N*HO*WO, KH*KW*C) with K ordered (ry, rx, rc) as the reference reduces."""
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    N, H, W, C = x.shape
    HO = conv_out_extent(H, KH, sh, pad, dh)
    WO = conv_out_extent(W, KW, sw, pad, dw)
    xp = np.zeros((N, H + 2 * pad, W + 2 * pad, C), dtype=x.dtype)
    xp[:, pad:pad + H, pad:pad + W, :] = x
    cols = np.empty((N, HO, WO, KH, KW, C), dtype=x.dtype)
    for ry in range(KH):
        for rx in range(KW):
            cols[:, :, :, ry, rx, :] = xp[:, ry * dh: ry * dh + (HO - 1) * sh + 1: sh,
                                          rx * dw: rx * dw + (WO - 1) * sw + 1: sw, :]
    return cols.reshape(N * HO * WO, KH * KW * C), (N, HO, WO)


def conv2d_nhwc_int(x, w, stride=1, pad=0, dilation=1):
    """uint8/int8 NHWC input, HWIO filter, int32 output; ops/cuda/conv2d.py:168-196."""
    KH, KW, CI, CO = w.shape
    cols, (N, HO, WO) = _im2col(x, KH, KW, stride, pad, dilation)
    out = _as_i64(cols) @ _as_i64(w).reshape(KH * KW * CI, CO)
    return _to_i32(out).reshape(N, HO, WO, CO)


def conv2d_nhwc_f16(x, w, stride=1, pad=0, dilation=1, out_dtype=np.float32):
    """fp16 NHWC conv with float64 accumulation; rounded to float32, then to fp16 if asked."""
    assert x.dtype == np.float16 and w.dtype == np.float16
    KH, KW, CI, CO = w.shape
    cols, (N, HO, WO) = _im2col(x, KH, KW, stride, pad, dilation)
    out = cols.astype(np.float64) @ w.astype(np.float64).reshape(KH * KW * CI, CO)
    out = out.astype(np.float32).reshape(N, HO, WO, CO)
    return out.astype(np.float16) if np.dtype(out_dtype) == np.float16 else out


def pack_filter_x86(w_hwio, sco=64, sci=4):
    """HWIO int8 filter -> the x86 operator's (CO/sco, KH, KW, CI/sci, sco, sci) layout
    (ops/x86/conv2d_int8.py:36-50)."""
    KH, KW, CI, CO = w_hwio.shape
    assert CO % sco == 0 and CI % sci == 0
    w = w_hwio.reshape(KH, KW, CI // sci, sci, CO // sco, sco)
    return np.ascontiguousarray(w.transpose(4, 0, 1, 2, 5, 3))


def unpack_filter_x86(w_packed):
    """Inverse of pack_filter_x86."""
    OC, KH, KW, IC, sco, sci = w_packed.shape
    w = w_packed.transpose(1, 2, 3, 5, 0, 4)
    return np.ascontiguousarray(w.reshape(KH, KW, IC * sci, OC * sco))


def conv2d_nhwc_packed(x, w_packed, stride=1, pad=0, dilation=1):
    """The x86 operator: uint8 input, packed int8 filter, int32 output (N,HO,WO,CO/sco,sco);
    ops/x86/conv2d_int8.py:74-93."""
    OC, KH, KW, IC, sco, sci = w_packed.shape
    out = conv2d_nhwc_int(x, unpack_filter_x86(w_packed), stride, pad, dilation)
    N, HO, WO, CO = out.shape
    return out.reshape(N, HO, WO, OC, sco)


def _nchw_im2col(x, w, stride, pad):
    """The reference's own lowering of the NCHW operator (ops/cuda/conv2d.py:51-86): pad the
    input, build A[MM, MK] with MM = N*HO*WO rows and MK = CI*KH*KW columns ordered (ci, kh, kw),
    B[CO, MK] from the OIHW filter; C = B . A^T; output[n, c, p, q] = C[c, n*HO*WO + p*WO + q]."""
    sh, sw = _pair(stride)
    N, CI, H, W = x.shape
    CO, _, KH, KW = w.shape
    HO = conv_out_extent(H, KH, sh, pad, 1)
    WO = conv_out_extent(W, KW, sw, pad, 1)
    xp = np.zeros((N, CI, H + 2 * pad, W + 2 * pad), dtype=x.dtype)
    xp[:, :, pad:pad + H, pad:pad + W] = x
    A = np.empty((N, HO, WO, CI, KH, KW), dtype=x.dtype)
    for kh in range(KH):
        for kw in range(KW):
            A[:, :, :, :, kh, kw] = xp[:, :, kh: kh + (HO - 1) * sh + 1: sh,
                                       kw: kw + (WO - 1) * sw + 1: sw].transpose(0, 2, 3, 1)
    return A.reshape(N * HO * WO, CI * KH * KW), w.reshape(CO, CI * KH * KW), (N, CO, HO, WO)


def conv2d_nchw_int(x, w, stride=1, pad=0):
    """uint8/int8 NCHW input, OIHW filter, int32 NCHW output (ops/cuda/conv2d.py:9-101)."""
    A, B, (N, CO, HO, WO) = _nchw_im2col(x, w, stride, pad)
    C = _to_i32(_as_i64(B) @ _as_i64(A).T)
    return np.ascontiguousarray(C.reshape(CO, N, HO, WO).transpose(1, 0, 2, 3))


def conv2d_nchw_f16(x, w, stride=1, pad=0, out_dtype=np.float32):
    assert x.dtype == np.float16 and w.dtype == np.float16
    A, B, (N, CO, HO, WO) = _nchw_im2col(x, w, stride, pad)
    C = (B.astype(np.float64) @ A.astype(np.float64).T).astype(np.float32)
    out = np.ascontiguousarray(C.reshape(CO, N, HO, WO).transpose(1, 0, 2, 3))
    return out.astype(np.float16) if np.dtype(out_dtype) == np.float16 else out


def gemv(a, x, out_dtype=None):
    """The tensor-core gemv exactly as the reference builds it (ops/cuda/gemv.py:12-30): pad the
    vector to an (8, K) matrix of zeros, multiply; out (M, 8)."""
    M, K = a.shape
    bpad = np.zeros((8, K), dtype=x.dtype)
    bpad[0] = x[0]
    if a.dtype == np.float16:
        out = (a.astype(np.float64) @ bpad.astype(np.float64).T).astype(np.float32)
        return out.astype(np.float16) if out_dtype is not None and np.dtype(out_dtype) == np.float16 else out
    return _to_i32(_as_i64(a) @ _as_i64(bpad).T)


def _ncw_im2col(x, w, stride, pad):
    """The reference's lowering (ops/cuda/conv1d.py:27-69): A[N*W_O, CI*KW] with columns ordered
    (ci, kw), B[CO, CI*KW]; C = B . A^T; output[n, c, q] = C[c, n*W_O + q]."""
    N, CI, W = x.shape
    CO, _, KW = w.shape
    WO = (W - KW + 2 * pad) // stride + 1
    xp = np.zeros((N, CI, W + 2 * pad), dtype=x.dtype)
    xp[:, :, pad:pad + W] = x
    A = np.empty((N, WO, CI, KW), dtype=x.dtype)
    for kw in range(KW):
        A[:, :, :, kw] = xp[:, :, kw: kw + (WO - 1) * stride + 1: stride].transpose(0, 2, 1)
    return A.reshape(N * WO, CI * KW), w.reshape(CO, CI * KW), (N, CO, WO)


def conv1d_ncw(x, w, stride=1, pad=0, out_dtype=None):
    A, B, (N, CO, WO) = _ncw_im2col(x, w, stride, pad)
    if x.dtype == np.float16:
        C = (B.astype(np.float64) @ A.astype(np.float64).T).astype(np.float32)
    else:
        C = _to_i32(_as_i64(B) @ _as_i64(A).T)
    out = np.ascontiguousarray(C.reshape(CO, N, WO).transpose(1, 0, 2))
    return out.astype(np.float16) if out_dtype is not None and np.dtype(out_dtype) == np.float16 else out


def pack_filter_x86_1d(w_wio, sco=64, sci=4):
    """(KW, CI, CO) int8 filter -> (CO/sco, KW, CI/sci, sco, sci) (ops/x86/conv1d_int8.py:48)."""
    return pack_filter_x86(w_wio[None], sco, sci)[:, 0]


def conv1d_nwc_packed(x, w_packed, stride=1, pad=0, dilation=1):
    """ops/x86/conv1d_int8.py:53-84 through the 2-D oracle with a height of one: the input is
    padded along the width here, so the 2-D call runs unpadded."""
    N, W, CI = x.shape
    xp = np.zeros((N, 1, W + 2 * pad, CI), dtype=x.dtype)
    xp[:, 0, pad:pad + W] = x
    out = conv2d_nhwc_packed(xp, w_packed[:, None], (1, stride), 0, (1, dilation))
    return out[:, 0]


def scan(a, N, out_dtype=None):
    """The reference's scan as it is written there: a product with the constant (N, K) matrix
    B[i, j] = 0 if i <= j else 1 (ops/cuda/scan.py:6-23)."""
    M, K = a.shape
    b = (np.arange(N)[:, None] > np.arange(K)[None, :])
    if a.dtype == np.float16:
        out = (a.astype(np.float64) @ b.astype(np.float64).T).astype(np.float32)
        return out.astype(np.float16) if out_dtype is not None and np.dtype(out_dtype) == np.float16 else out
    return _to_i32(_as_i64(a) @ b.astype(np.int64).T)


def t2d_nchw_stride1(x, w, padding, out_dtype=None):
    """The reference's "transposed" NCHW conv for stride 1, staged as it stages it
    (ops/cuda/conv2d_transposed.py:82-135): pad the input by K-1-padding zeros on every side, build
    A[N*H_O*W_O, CI*KH*KW] with A[i, (ci,kh,kw)] = Padded[n, ci, p+kh, q+kw], B[CO, CI*KH*KW] from
    the filter as stored, C = B . A^T, output[n, c, p, q] = C[c, n*H_O*W_O + p*W_O + q]."""
    N, CI, H, W = x.shape
    CO, _, KH, KW = w.shape
    ph, pw = KH - 1 - padding, KW - 1 - padding
    HO, WO = H - 2 * padding + KH - 1, W - 2 * padding + KW - 1
    xp = np.zeros((N, CI, H + 2 * ph, W + 2 * pw), dtype=x.dtype)
    xp[:, :, ph:ph + H, pw:pw + W] = x
    A = np.empty((N, HO, WO, CI, KH, KW), dtype=x.dtype)
    for kh in range(KH):
        for kw in range(KW):
            A[:, :, :, :, kh, kw] = xp[:, :, kh:kh + HO, kw:kw + WO].transpose(0, 2, 3, 1)
    A = A.reshape(N * HO * WO, CI * KH * KW)
    B = w.reshape(CO, CI * KH * KW)
    if x.dtype == np.float16:
        C = (B.astype(np.float64) @ A.astype(np.float64).T).astype(np.float32)
    else:
        C = _to_i32(_as_i64(B) @ _as_i64(A).T)
    out = np.ascontiguousarray(C.reshape(CO, N, HO, WO).transpose(1, 0, 2, 3))
    return out.astype(np.float16) if out_dtype is not None and np.dtype(out_dtype) == np.float16 else out


def conv3d_ncdhw(x, w, stride=1, pad=0, out_dtype=None):
    """The reference's lowering of the NCDHW operator (ops/cuda/conv3d.py:33-85): pad, build
    A[N*D_O*H_O*W_O, CI*KD*KH*KW] with columns ordered (ci, kd, kh, kw), B[CO, CI*KD*KH*KW];
    C = B . A^T; output[n, c, d, p, q] = C[c, ((n*D_O + d)*H_O + p)*W_O + q]."""
    sd, sh, sw = (stride, stride, stride) if isinstance(stride, int) else tuple(int(v) for v in stride)
    N, CI, D, H, W = x.shape
    CO, _, KD, KH, KW = w.shape
    DO, HO, WO = (D - KD + 2 * pad) // sd + 1, (H - KH + 2 * pad) // sh + 1, (W - KW + 2 * pad) // sw + 1
    xp = np.zeros((N, CI, D + 2 * pad, H + 2 * pad, W + 2 * pad), dtype=x.dtype)
    xp[:, :, pad:pad + D, pad:pad + H, pad:pad + W] = x
    A = np.empty((N, DO, HO, WO, CI, KD, KH, KW), dtype=x.dtype)
    for kd in range(KD):
        for kh in range(KH):
            for kw in range(KW):
                A[..., kd, kh, kw] = xp[:, :, kd:kd + (DO - 1) * sd + 1:sd, kh:kh + (HO - 1) * sh + 1:sh,
                                        kw:kw + (WO - 1) * sw + 1:sw].transpose(0, 2, 3, 4, 1)
    A = A.reshape(N * DO * HO * WO, CI * KD * KH * KW)
    B = w.reshape(CO, CI * KD * KH * KW)
    if x.dtype == np.float16:
        C = (B.astype(np.float64) @ A.astype(np.float64).T).astype(np.float32)
    else:
        C = _to_i32(_as_i64(B) @ _as_i64(A).T)
    out = np.ascontiguousarray(C.reshape(CO, N, DO, HO, WO).transpose(1, 0, 2, 3, 4))
    return out.astype(np.float16) if out_dtype is not None and np.dtype(out_dtype) == np.float16 else out
