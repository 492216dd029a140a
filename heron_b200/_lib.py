"""ctypes binding of libheron_b200.so (the C ABI declared in include/heron_b200.h).

The shared library is built in-tree by ``heron_b200.build`` and is the only compute path of the
package: if it is missing, loading fails with an error that says how to build it, and nothing
falls back to another implementation.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libheron_b200.so")

HB_OK = 0
HB_ERR_SHAPE = 1
HB_ERR_ALIGN = 2
HB_ERR_KNOB = 3
HB_ERR_LAUNCH = 4
HB_ERR_TIMEOUT = 5
HB_ERR_DEVICE = 6
HB_ERR_DTYPE = 7
HB_ERR_SCRATCH = 8
HB_ERR_STATIC_SCRATCH = 9

# hb_dtype
HB_F16, HB_F32, HB_S8, HB_U8, HB_S32 = 0, 1, 2, 3, 4

DTYPE_CODES = {
    "float16": HB_F16,
    "float32": HB_F32,
    "int8": HB_S8,
    "uint8": HB_U8,
    "int32": HB_S32,
}

# Every symbol include/heron_b200.h declares; the CPU test-suite checks the library exports them.
EXPORTED_SYMBOLS = (
    "hb_kernel_limits",
    "hb_version",
    "hb_sm_count",
    "hb_default_knobs",
    "hb_check_knobs",
    "hb_balanced_run",
    "hb_balanced_pieces",
    "hb_gemm",
    "hb_bmm",
    "hb_conv2d_nhwc",
    "hb_conv2d_packed_scratch_bytes",
    "hb_conv2d_nhwc_packed",
    "hb_conv2d_nchw_scratch_bytes",
    "hb_conv2d_nchw",
    "hb_plan_conv2d_nchw",
    "hb_gemv",
    "hb_scan_scratch_bytes",
    "hb_conv3d_ncdhw_scratch_bytes",
    "hb_conv3d_ncdhw",
    "hb_plan_conv3d_ncdhw",
    "hb_scan",
    "hb_plan_scan",
    "hb_conv1d_ncw_scratch_bytes",
    "hb_conv1d_ncw",
    "hb_conv1d_nwc_packed",
    "hb_plan_gemv",
    "hb_plan_conv1d_ncw",
    "hb_plan_conv1d_nwc_packed",
    "hb_conv2d_packed_noalloc_max_bytes",
    "hb_conv2d_nhwc_packed_noalloc",
    "hb_plan_gemm",
    "hb_plan_bmm",
    "hb_plan_conv2d_nhwc",
    "hb_plan_conv2d_nhwc_packed",
    "hb_plan_launch",
    "hb_plan_knobs",
    "hb_plan_set_peer_outputs",
    "hb_plan_destroy",
    "hb_last_status",
    "hb_status_string",
)


class HbKnobs(ctypes.Structure):
    """Mirror of ``hb_knobs``; zero means "library default"."""

    _fields_ = [
        ("tile_n", ctypes.c_int),
        ("stages", ctypes.c_int),
        ("swizzle_bytes", ctypes.c_int),
        ("acc_stages", ctypes.c_int),
        ("raster", ctypes.c_int),
        ("epilogue", ctypes.c_int),
        ("max_ctas", ctypes.c_int),
        ("cta_group", ctypes.c_int),
        ("l2_prefetch", ctypes.c_int),
        ("conv_algo", ctypes.c_int),
        ("tail_split", ctypes.c_int),
        ("split_k", ctypes.c_int),
        ("k_slices", ctypes.c_int),
        ("balance", ctypes.c_int),
        ("epi_warps", ctypes.c_int),
        ("silent_producer", ctypes.c_int),
        ("probe", ctypes.c_int),
    ]

    FIELDS = ("tile_n", "stages", "swizzle_bytes", "acc_stages", "raster", "epilogue", "max_ctas",
              "cta_group", "l2_prefetch", "conv_algo", "tail_split", "split_k", "k_slices", "balance", "epi_warps",
              "silent_producer", "probe")

    @classmethod
    def from_dict(cls, d):
        k = cls()
        for name in cls.FIELDS:
            setattr(k, name, int((d or {}).get(name, 0)))
        return k

    def to_dict(self):
        return {name: int(getattr(self, name)) for name in self.FIELDS}


class HbLimits(ctypes.Structure):
    """Mirror of ``hb_limits``."""

    _fields_ = [(n, ctypes.c_int) for n in
                ("max_shared_memory_per_block", "tmem_columns", "tile_m", "max_stages",
                 "epilogue_staging_bytes", "smem_slack_bytes", "static_scratch_bytes", "reserved")]


def kernel_limits():
    """The library's own SM limits as a dict (needs the built library, not a GPU)."""
    lim = HbLimits()
    check(load().hb_kernel_limits(ctypes.byref(lim)), "hb_kernel_limits")
    return {n: int(getattr(lim, n)) for n, _ in HbLimits._fields_ if n != "reserved"}


class HeronB200Error(RuntimeError):
    """A non-zero status from the library (the stand-in for the reference's TVMError)."""

    def __init__(self, status, where):
        self.status = status
        super().__init__("%s: status %d (%s)" % (where, status, status_string(status)))


_lib = None


def load():
    """Loads the shared library once and declares the argument types of every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libheron_b200.so is not built: run `python -m heron_b200.build` "
            "(needs nvcc with sm_100a support); there is no fallback path"
        )
    lib = ctypes.CDLL(LIB_PATH)
    c_int, c_void_p, c_size_t = ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t
    kp = ctypes.POINTER(HbKnobs)
    ip = ctypes.POINTER(c_int)
    lib.hb_version.restype = c_int
    lib.hb_version.argtypes = []
    lib.hb_kernel_limits.restype = c_int
    lib.hb_kernel_limits.argtypes = [ctypes.POINTER(HbLimits)]
    lib.hb_sm_count.restype = c_int
    lib.hb_sm_count.argtypes = []
    lib.hb_default_knobs.restype = c_int
    lib.hb_default_knobs.argtypes = [c_int] * 6 + [c_int, c_int, kp]
    lib.hb_check_knobs.restype = c_int
    lib.hb_check_knobs.argtypes = [c_int] * 6 + [c_int, c_int, kp, ip, ip]
    lib.hb_balanced_run.restype = c_int
    lib.hb_balanced_run.argtypes = [c_int] * 4 + [ip, ip]
    lib.hb_balanced_pieces.restype = c_int
    lib.hb_balanced_pieces.argtypes = [c_int] * 4 + [ip, c_int]
    lib.hb_gemm.restype = c_int
    lib.hb_gemm.argtypes = [c_void_p] * 3 + [c_int] * 3 + [c_int] * 3 + [kp, c_void_p]
    lib.hb_bmm.restype = c_int
    lib.hb_bmm.argtypes = [c_void_p] * 3 + [c_int] * 4 + [c_int] * 3 + [kp, c_void_p]
    lib.hb_conv2d_nhwc.restype = c_int
    lib.hb_conv2d_nhwc.argtypes = [c_void_p] * 3 + [c_int] * 12 + [c_int] * 3 + [kp, c_void_p]
    lib.hb_conv2d_packed_scratch_bytes.restype = c_size_t
    lib.hb_conv2d_packed_scratch_bytes.argtypes = [c_int] * 4
    lib.hb_conv2d_nhwc_packed.restype = c_int
    lib.hb_conv2d_nhwc_packed.argtypes = (
        [c_void_p] * 3 + [c_int] * 12 + [c_int, c_void_p, c_size_t, kp, c_void_p]
    )
    lib.hb_conv2d_packed_noalloc_max_bytes.restype = c_size_t
    lib.hb_conv2d_packed_noalloc_max_bytes.argtypes = []
    lib.hb_conv2d_nhwc_packed_noalloc.restype = c_int
    lib.hb_conv2d_nhwc_packed_noalloc.argtypes = [c_void_p] * 3 + [c_int] * 12 + [c_int, kp, c_void_p]
    lib.hb_conv2d_nchw_scratch_bytes.restype = c_size_t
    lib.hb_conv2d_nchw_scratch_bytes.argtypes = [c_int] * 10 + [c_int, c_int]
    lib.hb_conv2d_nchw.restype = c_int
    lib.hb_conv2d_nchw.argtypes = [c_void_p] * 3 + [c_int] * 10 + [c_int] * 3 + [c_void_p, c_size_t, kp, c_void_p]
    pp = ctypes.POINTER(c_void_p)
    lib.hb_plan_conv2d_nchw.restype = c_int
    lib.hb_plan_conv2d_nchw.argtypes = [pp] + lib.hb_conv2d_nchw.argtypes[:-1]
    lib.hb_gemv.restype = c_int
    lib.hb_gemv.argtypes = [c_void_p] * 3 + [c_int] * 2 + [c_int] * 3 + [kp, c_void_p]
    lib.hb_conv1d_ncw_scratch_bytes.restype = c_size_t
    lib.hb_conv1d_ncw_scratch_bytes.argtypes = [c_int] * 7 + [c_int, c_int]
    lib.hb_conv1d_ncw.restype = c_int
    lib.hb_conv1d_ncw.argtypes = [c_void_p] * 3 + [c_int] * 7 + [c_int] * 3 + [c_void_p, c_size_t, kp, c_void_p]
    lib.hb_conv1d_nwc_packed.restype = c_int
    lib.hb_conv1d_nwc_packed.argtypes = [c_void_p] * 3 + [c_int] * 8 + [c_int, c_void_p, c_size_t, kp, c_void_p]
    lib.hb_conv3d_ncdhw_scratch_bytes.restype = c_size_t
    lib.hb_conv3d_ncdhw_scratch_bytes.argtypes = [c_int] * 13 + [c_int, c_int]
    lib.hb_conv3d_ncdhw.restype = c_int
    lib.hb_conv3d_ncdhw.argtypes = [c_void_p] * 3 + [c_int] * 13 + [c_int] * 3 + [c_void_p, c_size_t, kp, c_void_p]
    lib.hb_plan_conv3d_ncdhw.restype = c_int
    lib.hb_plan_conv3d_ncdhw.argtypes = [pp] + lib.hb_conv3d_ncdhw.argtypes[:-1]
    lib.hb_scan_scratch_bytes.restype = c_size_t
    lib.hb_scan_scratch_bytes.argtypes = [c_int, c_int, c_int]
    lib.hb_scan.restype = c_int
    lib.hb_scan.argtypes = [c_void_p] * 2 + [c_int] * 3 + [c_int] * 2 + [c_void_p, c_size_t, kp, c_void_p]
    lib.hb_plan_scan.restype = c_int
    lib.hb_plan_scan.argtypes = [pp] + lib.hb_scan.argtypes[:-1]
    lib.hb_plan_gemv.restype = c_int
    lib.hb_plan_gemv.argtypes = [pp] + lib.hb_gemv.argtypes[:-1]
    lib.hb_plan_conv1d_ncw.restype = c_int
    lib.hb_plan_conv1d_ncw.argtypes = [pp] + lib.hb_conv1d_ncw.argtypes[:-1]
    lib.hb_plan_conv1d_nwc_packed.restype = c_int
    lib.hb_plan_conv1d_nwc_packed.argtypes = [pp] + lib.hb_conv1d_nwc_packed.argtypes[:-1]
    lib.hb_plan_gemm.restype = c_int
    lib.hb_plan_gemm.argtypes = [pp] + lib.hb_gemm.argtypes[:-1]
    lib.hb_plan_bmm.restype = c_int
    lib.hb_plan_bmm.argtypes = [pp] + lib.hb_bmm.argtypes[:-1]
    lib.hb_plan_conv2d_nhwc.restype = c_int
    lib.hb_plan_conv2d_nhwc.argtypes = [pp] + lib.hb_conv2d_nhwc.argtypes[:-1]
    lib.hb_plan_conv2d_nhwc_packed.restype = c_int
    lib.hb_plan_conv2d_nhwc_packed.argtypes = [pp] + lib.hb_conv2d_nhwc_packed.argtypes[:-1]
    lib.hb_plan_launch.restype = c_int
    lib.hb_plan_launch.argtypes = [c_void_p, c_void_p]
    lib.hb_plan_knobs.restype = c_int
    lib.hb_plan_knobs.argtypes = [c_void_p, kp, ip, ip]
    lib.hb_plan_set_peer_outputs.restype = c_int
    lib.hb_plan_set_peer_outputs.argtypes = [c_void_p, c_int, ctypes.POINTER(c_void_p)]
    lib.hb_plan_destroy.restype = None
    lib.hb_plan_destroy.argtypes = [c_void_p]
    lib.hb_last_status.restype = c_int
    lib.hb_last_status.argtypes = [ip]
    lib.hb_status_string.restype = ctypes.c_char_p
    lib.hb_status_string.argtypes = [c_int]
    _lib = lib
    return lib


def status_string(status):
    try:
        return load().hb_status_string(int(status)).decode()
    except ImportError:
        return "library not built"


def check(status, where):
    if status != HB_OK:
        raise HeronB200Error(status, where)


def last_status():
    """Synchronises the device and returns (then clears) the kernels' status word."""
    v = ctypes.c_int(0)
    check(load().hb_last_status(ctypes.byref(v)), "hb_last_status")
    return v.value
