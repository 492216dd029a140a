"""Device-tensor front end of the C ABI: torch tensors in, torch tensors out.

torch is used for device memory and streams only; every function here hands raw device pointers
to libheron_b200.so and raises ``HeronB200Error`` on a non-zero status.  Operand conventions are
the reference operators' own: GEMM / batched GEMM take ``B`` as (N, K) (ops/cuda/dense.py:6,
ops/cuda/batch_matmul.py:8), NHWC conv takes an HWIO filter (ops/cuda/conv2d.py:155).
"""
import ctypes

import torch

from . import _lib

_TORCH_CODES = {
    torch.float16: _lib.HB_F16,
    torch.float32: _lib.HB_F32,
    torch.int8: _lib.HB_S8,
    torch.uint8: _lib.HB_U8,
    torch.int32: _lib.HB_S32,
}

TORCH_DTYPES = {
    "float16": torch.float16,
    "float32": torch.float32,
    "int8": torch.int8,
    "uint8": torch.uint8,
    "int32": torch.int32,
}


def _code(t):
    try:
        return _TORCH_CODES[t.dtype]
    except KeyError:
        raise _lib.HeronB200Error(_lib.HB_ERR_DTYPE, "dtype %s" % t.dtype)


def _dev(t, name):
    if not t.is_cuda:
        raise ValueError("%s must be a CUDA tensor: the kernels have no CPU path" % name)
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    return ctypes.c_void_p(t.data_ptr())


def _out(out, shape, like, name="out"):
    """A caller-supplied output must be exactly what the kernel will write: a wrong size would put
    stores past the end of the buffer."""
    if tuple(out.shape) != tuple(shape):
        raise ValueError("%s has shape %s, the operator writes %s" % (name, tuple(out.shape), tuple(shape)))
    if out.dtype not in _TORCH_CODES:
        raise _lib.HeronB200Error(_lib.HB_ERR_DTYPE, "dtype %s" % out.dtype)
    if out.device != like.device:
        raise ValueError("%s is on %s, the inputs are on %s" % (name, out.device, like.device))
    return out


def _same_device(*tensors):
    """All operands on one device, and that device current: the library launches on the current
    CUDA device, so a tensor elsewhere would hand it a pointer of another GPU."""
    dev = tensors[0].device
    for t in tensors:
        if t.device != dev:
            raise ValueError("operands live on different devices: %s and %s" % (dev, t.device))
    if dev.type == "cuda" and dev.index is not None and dev.index != torch.cuda.current_device():
        raise ValueError("tensors are on cuda:%d but the current device is cuda:%d; wrap the call in "
                         "torch.cuda.device(...)" % (dev.index, torch.cuda.current_device()))


def _bytes_buf(buf, need, like, name):
    if buf.numel() * buf.element_size() < need:
        raise ValueError("%s holds %d bytes, the operator needs %d" % (name, buf.numel() * buf.element_size(), need))
    if buf.device != like.device:
        raise ValueError("%s is on %s, the inputs are on %s" % (name, buf.device, like.device))
    return buf


def _knobs(knobs):
    if knobs is None:
        return None
    if isinstance(knobs, _lib.HbKnobs):
        return ctypes.byref(knobs)
    return ctypes.byref(_lib.HbKnobs.from_dict(knobs))


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def default_out_dtype(in_dtype):
    return torch.float32 if in_dtype == torch.float16 else torch.int32


def gemm(a, b, out=None, out_dtype=None, knobs=None):
    """out[M,N] = sum_k a[M,k] * b[N,k]."""
    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise ValueError("a is (M,K), b is (N,K): K differs")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or default_out_dtype(a.dtype), device=a.device)
    _same_device(a, b, _out(out, (M, N), a))
    rc = _lib.load().hb_gemm(_dev(a, "a"), _dev(b, "b"), _dev(out, "out"), M, K, N, _code(a),
                             _code(b), _code(out), _knobs(knobs), _stream(a))
    _lib.check(rc, "hb_gemm")
    return out


def bmm(a, b, out=None, out_dtype=None, knobs=None):
    """out[b,M,N] = sum_k a[b,M,k] * b[b,N,k]."""
    B, M, K = a.shape
    B2, N, K2 = b.shape
    if K != K2 or B != B2:
        raise ValueError("a is (B,M,K), b is (B,N,K): shapes differ")
    if out is None:
        out = torch.empty((B, M, N), dtype=out_dtype or default_out_dtype(a.dtype), device=a.device)
    _same_device(a, b, _out(out, (B, M, N), a))
    rc = _lib.load().hb_bmm(_dev(a, "a"), _dev(b, "b"), _dev(out, "out"), B, M, K, N, _code(a),
                            _code(b), _code(out), _knobs(knobs), _stream(a))
    _lib.check(rc, "hb_bmm")
    return out


def _pair(v):
    if isinstance(v, int):
        return v, v
    a, b = v
    return int(a), int(b)


def conv_out_hw(H, W, KH, KW, stride, padding, dilation):
    """Output extent of the reference's NHWC conv (ops/cuda/conv2d.py:165-175)."""
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    HO = (H - ((KH - 1) * dh + 1) + 2 * padding) // sh + 1
    WO = (W - ((KW - 1) * dw + 1) + 2 * padding) // sw + 1
    if HO <= 0 or WO <= 0:
        # the window does not fit the padded image: the library's own answer, before any allocation
        raise _lib.HeronB200Error(_lib.HB_ERR_SHAPE, "conv output extent %d x %d" % (HO, WO))
    return HO, WO


def conv2d_nhwc(x, w, stride=1, padding=0, dilation=1, out=None, out_dtype=None, knobs=None):
    """out[n,y,x,f] = sum pad(x)[n, y*s+ry*d, x*s+rx*d, c] * w[ry,rx,c,f]; w is HWIO."""
    N, H, W, CI = x.shape
    KH, KW, CI2, CO = w.shape
    if CI != CI2:
        raise ValueError("input channels of x and w differ")
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    HO, WO = conv_out_hw(H, W, KH, KW, stride, padding, dilation)
    if out is None:
        out = torch.empty((N, HO, WO, CO), dtype=out_dtype or default_out_dtype(x.dtype),
                          device=x.device)
    _same_device(x, w, _out(out, (N, HO, WO, CO), x))
    rc = _lib.load().hb_conv2d_nhwc(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), N, H, W, CI, CO,
                                    KH, KW, sh, sw, int(padding), dh, dw, _code(x), _code(w),
                                    _code(out), _knobs(knobs), _stream(x))
    _lib.check(rc, "hb_conv2d_nhwc")
    return out


def conv2d_nhwc_packed(x, w_packed, CO, KH, KW, stride=1, padding=0, dilation=1, sco=64, out=None,
                       scratch=None, knobs=None):
    """The x86 operator's conv: uint8 NHWC input, int8 filter packed (CO/sco,KH,KW,CI/4,sco,4)."""
    N, H, W, CI = x.shape
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    HO, WO = conv_out_hw(H, W, KH, KW, stride, padding, dilation)
    lib = _lib.load()
    need = lib.hb_conv2d_packed_scratch_bytes(CI, CO, KH, KW)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.int8, device=x.device)
    if out is None:
        out = torch.empty((N, HO, WO, CO // sco, sco), dtype=torch.int32, device=x.device)
    _packed_checks(x, w_packed, out, scratch, need, (N, HO, WO, CO // sco, sco), (CO // sco, KH, KW, CI // 4, sco, 4))
    rc = lib.hb_conv2d_nhwc_packed(_dev(x, "x"), _dev(w_packed, "w_packed"), _dev(out, "out"), N, H,
                                   W, CI, CO, KH, KW, sh, sw, int(padding), dh, dw, int(sco),
                                   _dev(scratch, "scratch"), scratch.numel(), _knobs(knobs),
                                   _stream(x))
    _lib.check(rc, "hb_conv2d_nhwc_packed")
    return out


def _packed_checks(x, w_packed, out, scratch, need, out_shape, w_shape):
    n_w = 1
    for d in w_shape:
        n_w *= d
    if w_packed.numel() != n_w or w_packed.element_size() != 1:
        raise ValueError("w_packed holds %d elements, the packed filter %s has %d" % (w_packed.numel(), w_shape, n_w))
    if tuple(out.shape) == out_shape[:3] + (out_shape[3] * out_shape[4],):
        out_shape = tuple(out.shape)  # (N, HO, WO, CO): the same bytes as (N, HO, WO, CO/sco, sco)
    _same_device(x, w_packed, _out(out, out_shape, x), _bytes_buf(scratch, need, x, "scratch"))


def _nchw_common(x, w, stride, padding, out, out_dtype, scratch):
    N, CI, H, W = x.shape
    CO, CI2, KH, KW = w.shape
    if CI != CI2:
        raise ValueError("input channels of x and w differ")
    sh, sw = _pair(stride)
    HO, WO = conv_out_hw(H, W, KH, KW, stride, padding, 1)
    if out is None:
        out = torch.empty((N, CO, HO, WO), dtype=out_dtype or default_out_dtype(x.dtype), device=x.device)
    need = _lib.load().hb_conv2d_nchw_scratch_bytes(N, H, W, CI, CO, KH, KW, sh, sw, int(padding), _code(x),
                                                   _code(out))
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    _same_device(x, w, _out(out, (N, CO, HO, WO), x), _bytes_buf(scratch, need, x, "scratch"))
    return (N, H, W, CI, CO, KH, KW, sh, sw, int(padding)), out, scratch


def conv2d_nchw(x, w, stride=1, padding=0, out=None, out_dtype=None, scratch=None, knobs=None):
    """out[n,c,p,q] = sum pad(x)[n,ci,p*s+kh,q*s+kw] * w[c,ci,kh,kw]; x NCHW, w OIHW, dilation 1."""
    dims, out, scratch = _nchw_common(x, w, stride, padding, out, out_dtype, scratch)
    rc = _lib.load().hb_conv2d_nchw(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), *dims, _code(x), _code(w),
                                    _code(out), _dev(scratch, "scratch"), scratch.numel(), _knobs(knobs),
                                    _stream(x))
    _lib.check(rc, "hb_conv2d_nchw")
    return out


def plan_conv2d_nchw(x, w, stride=1, padding=0, out=None, out_dtype=None, scratch=None, knobs=None):
    dims, out, scratch = _nchw_common(x, w, stride, padding, out, out_dtype, scratch)
    h = ctypes.c_void_p()
    rc = _lib.load().hb_plan_conv2d_nchw(ctypes.byref(h), _dev(x, "x"), _dev(w, "w"), _dev(out, "out"), *dims,
                                         _code(x), _code(w), _code(out), _dev(scratch, "scratch"),
                                         scratch.numel(), _knobs(knobs))
    _lib.check(rc, "hb_plan_conv2d_nchw")
    return Plan(h, (x, w, scratch), out)


class Plan:
    """A launch-ready kernel bound to fixed buffers (hb_plan): build once, launch many times.

    Keeps references to the tensors it was built on so that their memory outlives the plan.
    """

    def __init__(self, handle, tensors, out):
        self._handle = handle
        self._tensors = tensors
        self.out = out

    def launch(self, stream=None):
        if stream is None:
            stream = torch.cuda.current_stream(self.out.device).cuda_stream
        _lib.check(_lib.load().hb_plan_launch(self._handle, ctypes.c_void_p(stream)), "hb_plan_launch")
        return self.out

    __call__ = launch

    def knobs(self):
        """Resolved knobs plus the persistent grid size and dynamic shared memory of the launch."""
        k = _lib.HbKnobs()
        grid, smem = ctypes.c_int(0), ctypes.c_int(0)
        _lib.check(_lib.load().hb_plan_knobs(self._handle, ctypes.byref(k), ctypes.byref(grid),
                                             ctypes.byref(smem)), "hb_plan_knobs")
        d = k.to_dict()
        d["grid"], d["smem_bytes"] = grid.value, smem.value
        return d

    def set_peer_outputs(self, outs):
        """Every tile the kernel stores to this plan's output also goes to each tensor of `outs`
        (same shape, dtype and layout; typically this rank's slice of the other GPUs' output
        buffers, mapped into this process).  An empty list removes them."""
        outs = list(outs)
        for o in outs:
            if tuple(o.shape) != tuple(self.out.shape) or o.dtype != self.out.dtype or not o.is_contiguous():
                raise ValueError("a peer output must have the plan's output shape, dtype and a dense layout")
        arr = (ctypes.c_void_p * max(len(outs), 1))(*[o.data_ptr() for o in outs])
        _lib.check(_lib.load().hb_plan_set_peer_outputs(self._handle, len(outs), arr), "hb_plan_set_peer_outputs")
        self._peer_outs = outs  # (kept alive with the plan)

    def close(self):
        if self._handle is not None:
            _lib.load().hb_plan_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def plan_gemm(a, b, out=None, out_dtype=None, knobs=None):
    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise ValueError("a is (M,K), b is (N,K): K differs")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or default_out_dtype(a.dtype), device=a.device)
    _same_device(a, b, _out(out, (M, N), a))
    h = ctypes.c_void_p()
    rc = _lib.load().hb_plan_gemm(ctypes.byref(h), _dev(a, "a"), _dev(b, "b"), _dev(out, "out"), M,
                                  K, N, _code(a), _code(b), _code(out), _knobs(knobs))
    _lib.check(rc, "hb_plan_gemm")
    return Plan(h, (a, b), out)


def plan_bmm(a, b, out=None, out_dtype=None, knobs=None):
    B, M, K = a.shape
    B2, N, K2 = b.shape
    if K != K2 or B != B2:
        raise ValueError("a is (B,M,K), b is (B,N,K): shapes differ")
    if out is None:
        out = torch.empty((B, M, N), dtype=out_dtype or default_out_dtype(a.dtype), device=a.device)
    _same_device(a, b, _out(out, (B, M, N), a))
    h = ctypes.c_void_p()
    rc = _lib.load().hb_plan_bmm(ctypes.byref(h), _dev(a, "a"), _dev(b, "b"), _dev(out, "out"), B,
                                 M, K, N, _code(a), _code(b), _code(out), _knobs(knobs))
    _lib.check(rc, "hb_plan_bmm")
    return Plan(h, (a, b), out)


def plan_conv2d_nhwc(x, w, stride=1, padding=0, dilation=1, out=None, out_dtype=None, knobs=None):
    N, H, W, CI = x.shape
    KH, KW, CI2, CO = w.shape
    if CI != CI2:
        raise ValueError("input channels of x and w differ")
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    HO, WO = conv_out_hw(H, W, KH, KW, stride, padding, dilation)
    if out is None:
        out = torch.empty((N, HO, WO, CO), dtype=out_dtype or default_out_dtype(x.dtype),
                          device=x.device)
    _same_device(x, w, _out(out, (N, HO, WO, CO), x))
    h = ctypes.c_void_p()
    rc = _lib.load().hb_plan_conv2d_nhwc(ctypes.byref(h), _dev(x, "x"), _dev(w, "w"),
                                         _dev(out, "out"), N, H, W, CI, CO, KH, KW, sh, sw,
                                         int(padding), dh, dw, _code(x), _code(w), _code(out),
                                         _knobs(knobs))
    _lib.check(rc, "hb_plan_conv2d_nhwc")
    return Plan(h, (x, w), out)


def plan_conv2d_nhwc_packed(x, w_packed, CO, KH, KW, stride=1, padding=0, dilation=1, sco=64,
                            out=None, scratch=None, knobs=None):
    N, H, W, CI = x.shape
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    HO, WO = conv_out_hw(H, W, KH, KW, stride, padding, dilation)
    lib = _lib.load()
    need = lib.hb_conv2d_packed_scratch_bytes(CI, CO, KH, KW)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.int8, device=x.device)
    if out is None:
        out = torch.empty((N, HO, WO, CO // sco, sco), dtype=torch.int32, device=x.device)
    _packed_checks(x, w_packed, out, scratch, need, (N, HO, WO, CO // sco, sco), (CO // sco, KH, KW, CI // 4, sco, 4))
    h = ctypes.c_void_p()
    rc = lib.hb_plan_conv2d_nhwc_packed(ctypes.byref(h), _dev(x, "x"), _dev(w_packed, "w_packed"),
                                        _dev(out, "out"), N, H, W, CI, CO, KH, KW, sh, sw,
                                        int(padding), dh, dw, int(sco), _dev(scratch, "scratch"),
                                        scratch.numel(), _knobs(knobs))
    _lib.check(rc, "hb_plan_conv2d_nhwc_packed")
    return Plan(h, (x, w_packed, scratch), out)


# ---- operators next to the hot path that run on the same kernels ---------------------------
def _gemv_args(a, x, out, out_dtype):
    M, K = a.shape
    if tuple(x.shape) != (1, K):
        raise ValueError("a is (M,K), x is (1,K)")
    if out is None:
        out = torch.empty((M, 8), dtype=out_dtype or default_out_dtype(a.dtype), device=a.device)
    if tuple(out.shape) != (M, 8):
        raise ValueError("out is (M, 8): column 0 holds the product (ops/cuda/gemv.py:7)")
    return M, K, out


def gemv(a, x, out=None, out_dtype=None, knobs=None):
    """out[i,0] = sum_k a[i,k] * x[0,k]; out[i,1..7] = 0 (the reference's 8-row padded form)."""
    M, K, out = _gemv_args(a, x, out, out_dtype)
    rc = _lib.load().hb_gemv(_dev(a, "a"), _dev(x, "x"), _dev(out, "out"), M, K, _code(a), _code(x),
                             _code(out), _knobs(knobs), _stream(a))
    _lib.check(rc, "hb_gemv")
    return out


def plan_gemv(a, x, out=None, out_dtype=None, knobs=None):
    M, K, out = _gemv_args(a, x, out, out_dtype)
    h = ctypes.c_void_p()
    rc = _lib.load().hb_plan_gemv(ctypes.byref(h), _dev(a, "a"), _dev(x, "x"), _dev(out, "out"), M, K,
                                  _code(a), _code(x), _code(out), _knobs(knobs))
    _lib.check(rc, "hb_plan_gemv")
    return Plan(h, (a, x), out)


def conv1d_out_w(W, KW, stride, padding, dilation=1):
    """(W - dilated_KW + 2*pad) // stride + 1 (ops/cuda/conv1d.py:24-25, ops/x86/conv1d_int8.py:53-55)."""
    WO = (W - ((KW - 1) * dilation + 1) + 2 * padding) // stride + 1
    if WO <= 0:
        raise _lib.HeronB200Error(_lib.HB_ERR_SHAPE, "conv1d output extent %d" % WO)
    return WO


def _c1d_ncw_args(x, w, stride, padding, out, out_dtype, scratch):
    N, CI, W = x.shape
    CO, CI2, KW = w.shape
    if CI != CI2:
        raise ValueError("input channels of x and w differ")
    WO = conv1d_out_w(W, KW, int(stride), int(padding))
    if out is None:
        out = torch.empty((N, CO, WO), dtype=out_dtype or default_out_dtype(x.dtype), device=x.device)
    need = _lib.load().hb_conv1d_ncw_scratch_bytes(N, W, CI, CO, KW, int(stride), int(padding), _code(x),
                                                  _code(out))
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    return (N, W, CI, CO, KW, int(stride), int(padding)), out, scratch


def conv1d_ncw(x, w, stride=1, padding=0, out=None, out_dtype=None, scratch=None, knobs=None):
    """out[n,c,q] = sum pad(x)[n,ci,q*s+kw] * w[c,ci,kw]; x (N,CI,W), w (CO,CI,KW), dilation 1."""
    dims, out, scratch = _c1d_ncw_args(x, w, stride, padding, out, out_dtype, scratch)
    rc = _lib.load().hb_conv1d_ncw(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), *dims, _code(x), _code(w),
                                   _code(out), _dev(scratch, "scratch"), scratch.numel(), _knobs(knobs),
                                   _stream(x))
    _lib.check(rc, "hb_conv1d_ncw")
    return out


def plan_conv1d_ncw(x, w, stride=1, padding=0, out=None, out_dtype=None, scratch=None, knobs=None):
    dims, out, scratch = _c1d_ncw_args(x, w, stride, padding, out, out_dtype, scratch)
    h = ctypes.c_void_p()
    rc = _lib.load().hb_plan_conv1d_ncw(ctypes.byref(h), _dev(x, "x"), _dev(w, "w"), _dev(out, "out"), *dims,
                                        _code(x), _code(w), _code(out), _dev(scratch, "scratch"),
                                        scratch.numel(), _knobs(knobs))
    _lib.check(rc, "hb_plan_conv1d_ncw")
    return Plan(h, (x, w, scratch), out)


def _c1d_packed_args(x, CO, KW, stride, padding, dilation, sco, out, scratch):
    N, W, CI = x.shape
    WO = conv1d_out_w(W, KW, int(stride), int(padding), int(dilation))
    lib = _lib.load()
    if scratch is None:
        scratch = torch.empty(lib.hb_conv2d_packed_scratch_bytes(CI, CO, 1, KW), dtype=torch.int8,
                              device=x.device)
    if out is None:
        out = torch.empty((N, WO, CO // sco, sco), dtype=torch.int32, device=x.device)
    return (N, W, CI, CO, KW, int(stride), int(padding), int(dilation), int(sco)), out, scratch


def conv1d_nwc_packed(x, w_packed, CO, KW, stride=1, padding=0, dilation=1, sco=64, out=None,
                      scratch=None, knobs=None):
    """The x86 1-D conv: uint8 (N,W,CI) input, int8 filter packed (CO/sco, KW, CI/4, sco, 4)."""
    dims, out, scratch = _c1d_packed_args(x, CO, KW, stride, padding, dilation, sco, out, scratch)
    rc = _lib.load().hb_conv1d_nwc_packed(_dev(x, "x"), _dev(w_packed, "w_packed"), _dev(out, "out"), *dims,
                                          _dev(scratch, "scratch"), scratch.numel(), _knobs(knobs),
                                          _stream(x))
    _lib.check(rc, "hb_conv1d_nwc_packed")
    return out


def plan_conv1d_nwc_packed(x, w_packed, CO, KW, stride=1, padding=0, dilation=1, sco=64, out=None,
                           scratch=None, knobs=None):
    dims, out, scratch = _c1d_packed_args(x, CO, KW, stride, padding, dilation, sco, out, scratch)
    h = ctypes.c_void_p()
    rc = _lib.load().hb_plan_conv1d_nwc_packed(ctypes.byref(h), _dev(x, "x"), _dev(w_packed, "w_packed"),
                                               _dev(out, "out"), *dims, _dev(scratch, "scratch"),
                                               scratch.numel(), _knobs(knobs))
    _lib.check(rc, "hb_plan_conv1d_nwc_packed")
    return Plan(h, (x, w_packed, scratch), out)


def _scan_args(a, N, out, out_dtype, scratch):
    M, K = a.shape
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or default_out_dtype(a.dtype), device=a.device)
    if scratch is None:
        scratch = torch.empty(_lib.load().hb_scan_scratch_bytes(N, K, _code(a)), dtype=torch.uint8, device=a.device)
    return M, K, out, scratch


def scan(a, N, out=None, out_dtype=None, scratch=None, knobs=None):
    """out[m,n] = sum of a[m,k] over k < min(n, K): the reference's scan operator, a GEMM with the
    constant matrix B[n,k] = (n <= k) ? 0 : 1 (ops/cuda/scan.py:6-23)."""
    M, K, out, scratch = _scan_args(a, N, out, out_dtype, scratch)
    rc = _lib.load().hb_scan(_dev(a, "a"), _dev(out, "out"), M, N, K, _code(a), _code(out),
                             _dev(scratch, "scratch"), scratch.numel(), _knobs(knobs), _stream(a))
    _lib.check(rc, "hb_scan")
    return out


def plan_scan(a, N, out=None, out_dtype=None, scratch=None, knobs=None):
    M, K, out, scratch = _scan_args(a, N, out, out_dtype, scratch)
    h = ctypes.c_void_p()
    rc = _lib.load().hb_plan_scan(ctypes.byref(h), _dev(a, "a"), _dev(out, "out"), M, N, K, _code(a),
                                  _code(out), _dev(scratch, "scratch"), scratch.numel(), _knobs(knobs))
    _lib.check(rc, "hb_plan_scan")
    return Plan(h, (a, scratch), out)


def _triple(v):
    if isinstance(v, int):
        return v, v, v
    a, b, c = v
    return int(a), int(b), int(c)


def _c3d_args(x, w, stride, padding, out, out_dtype, scratch):
    N, CI, D, H, W = x.shape
    CO, CI2, KD, KH, KW = w.shape
    if CI != CI2:
        raise ValueError("input channels of x and w differ")
    sd, sh, sw = _triple(stride)
    p = int(padding)
    DO, HO, WO = (D - KD + 2 * p) // sd + 1, (H - KH + 2 * p) // sh + 1, (W - KW + 2 * p) // sw + 1
    if DO <= 0 or HO <= 0 or WO <= 0:
        raise _lib.HeronB200Error(_lib.HB_ERR_SHAPE, "conv3d output extent %d x %d x %d" % (DO, HO, WO))
    if out is None:
        out = torch.empty((N, CO, DO, HO, WO), dtype=out_dtype or default_out_dtype(x.dtype), device=x.device)
    dims = (N, D, H, W, CI, CO, KD, KH, KW, sd, sh, sw, p)
    need = _lib.load().hb_conv3d_ncdhw_scratch_bytes(*dims, _code(x), _code(out))
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    return dims, out, scratch


def conv3d_ncdhw(x, w, stride=1, padding=0, out=None, out_dtype=None, scratch=None, knobs=None):
    """out[n,c,d,p,q] = sum pad(x)[n,ci,d*sd+kd,p*sh+kh,q*sw+kw] * w[c,ci,kd,kh,kw]; x NCDHW, w OIDHW,
    dilation 1 (ops/cuda/conv3d.py:9-85)."""
    dims, out, scratch = _c3d_args(x, w, stride, padding, out, out_dtype, scratch)
    rc = _lib.load().hb_conv3d_ncdhw(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), *dims, _code(x), _code(w),
                                     _code(out), _dev(scratch, "scratch"), scratch.numel(), _knobs(knobs),
                                     _stream(x))
    _lib.check(rc, "hb_conv3d_ncdhw")
    return out


def plan_conv3d_ncdhw(x, w, stride=1, padding=0, out=None, out_dtype=None, scratch=None, knobs=None):
    dims, out, scratch = _c3d_args(x, w, stride, padding, out, out_dtype, scratch)
    h = ctypes.c_void_p()
    rc = _lib.load().hb_plan_conv3d_ncdhw(ctypes.byref(h), _dev(x, "x"), _dev(w, "w"), _dev(out, "out"), *dims,
                                          _code(x), _code(w), _code(out), _dev(scratch, "scratch"),
                                          scratch.numel(), _knobs(knobs))
    _lib.check(rc, "hb_plan_conv3d_ncdhw")
    return Plan(h, (x, w, scratch), out)
