"""The C ABI on a machine without a GPU: the library loads, exports every symbol the header
declares, answers the host-only queries, and refuses to compute (no CPU fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "heron_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hb_[a-z0-9_]+)\s*\(", text)))


def test_exports_match_header(hb_lib):
    from heron_b200 import _lib
    declared = header_symbols()
    assert declared, "no declarations found in include/heron_b200.h"
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared
    for name in declared:
        assert hasattr(hb_lib, name), name


def test_version_and_status_strings(hb_lib):
    from heron_b200 import _lib
    assert hb_lib.hb_version() >= 100
    for code in range(0, 9):
        assert _lib.status_string(code)
    assert "unknown" in _lib.status_string(99)


def test_default_knobs_are_inside_the_space(hb_lib):
    from heron_b200 import _lib
    cases = [
        (0, 1, 64, 64, 64, 64, _lib.HB_U8, _lib.HB_S32),
        (0, 1, 4096, 4096, 4096, 4096, _lib.HB_F16, _lib.HB_F32),
        (1, 192, 512, 512, 64, 64, _lib.HB_S8, _lib.HB_S32),
        (2, 1, 100352, 64, 576, 64, _lib.HB_F16, _lib.HB_F16),
        (2, 1, 50176, 512, 4608, 512, _lib.HB_U8, _lib.HB_S32),
        (2, 1, 324, 64, 144, 16, _lib.HB_F16, _lib.HB_F32),
    ]
    for op, batch, M, N, K, kin, tin, tout in cases:
        k = _lib.HbKnobs()
        assert hb_lib.hb_default_knobs(op, batch, M, N, K, kin, tin, tout, ctypes.byref(k)) == 0
        smem, cols = ctypes.c_int(0), ctypes.c_int(0)
        rc = hb_lib.hb_check_knobs(op, batch, M, N, K, kin, tin, tout, ctypes.byref(k),
                                   ctypes.byref(smem), ctypes.byref(cols))
        assert rc == 0, (op, M, N, K, k.to_dict())
        assert 0 < smem.value <= 232448 and cols.value in (32, 64, 128, 256, 512)
    # the quoted configuration keeps the widest tile
    k = _lib.HbKnobs()
    hb_lib.hb_default_knobs(0, 1, 4096, 4096, 4096, 4096, _lib.HB_F16, _lib.HB_F32, ctypes.byref(k))
    assert k.tile_n == 256 and k.swizzle_bytes == 128 and k.acc_stages == 2


@pytest.mark.parametrize("bad", [
    dict(tile_n=48), dict(tile_n=288), dict(stages=13), dict(swizzle_bytes=96),
    dict(tile_n=256, stages=12), dict(acc_stages=3), dict(raster=2), dict(epilogue=3), dict(cta_group=3),
    dict(l2_prefetch=65), dict(k_slices=3), dict(k_slices=2, stages=4),  # a ring of 4 x 2 x 32 KB plus the staging buffers
])
def test_check_knobs_rejects(hb_lib, bad):
    from heron_b200 import _lib
    k = _lib.HbKnobs.from_dict(bad)
    rc = hb_lib.hb_check_knobs(0, 1, 4096, 4096, 4096, 4096, _lib.HB_F16, _lib.HB_F32, ctypes.byref(k), None, None)
    assert rc == _lib.HB_ERR_KNOB


def test_fp16_output_needs_64_column_tiles(hb_lib):
    from heron_b200 import _lib
    k = _lib.HbKnobs.from_dict(dict(tile_n=96))
    assert hb_lib.hb_check_knobs(0, 1, 512, 512, 512, 512, _lib.HB_F16, _lib.HB_F16, ctypes.byref(k), None, None) == _lib.HB_ERR_KNOB
    assert hb_lib.hb_check_knobs(0, 1, 512, 512, 512, 512, _lib.HB_F16, _lib.HB_F32, ctypes.byref(k), None, None) == 0


def test_argument_errors_come_before_the_device(hb_lib):
    """Shape / dtype / alignment errors are reported without touching a GPU."""
    from heron_b200 import _lib
    buf = np.zeros(4096, dtype=np.uint8)
    p = ctypes.c_void_p(buf.ctypes.data & ~15)
    assert hb_lib.hb_gemm(p, p, p, 0, 64, 64, _lib.HB_U8, _lib.HB_S8, _lib.HB_S32, None, None) == _lib.HB_ERR_SHAPE
    assert hb_lib.hb_gemm(p, p, p, 64, 24, 64, _lib.HB_U8, _lib.HB_S8, _lib.HB_S32, None, None) == _lib.HB_ERR_SHAPE
    assert hb_lib.hb_gemm(p, p, p, 64, 64, 64, _lib.HB_F16, _lib.HB_S8, _lib.HB_S32, None, None) == _lib.HB_ERR_DTYPE
    assert hb_lib.hb_gemm(p, p, p, 64, 64, 64, _lib.HB_U8, _lib.HB_S8, _lib.HB_F32, None, None) == _lib.HB_ERR_DTYPE
    odd = ctypes.c_void_p((buf.ctypes.data & ~15) + 8)
    assert hb_lib.hb_gemm(odd, p, p, 64, 64, 64, _lib.HB_U8, _lib.HB_S8, _lib.HB_S32, None, None) == _lib.HB_ERR_ALIGN
    assert hb_lib.hb_gemm(None, p, p, 64, 64, 64, _lib.HB_U8, _lib.HB_S8, _lib.HB_S32, None, None) == _lib.HB_ERR_ALIGN
    # conv: channel bytes must be a multiple of 32, stride <= 8
    args = [p, p, p, 1, 8, 8, 8, 16, 3, 3, 1, 1, 1, 1, 1, _lib.HB_F16, _lib.HB_F16, _lib.HB_F32, None, None]
    assert hb_lib.hb_conv2d_nhwc(*args) == _lib.HB_ERR_SHAPE
    args[6] = 16
    args[10] = 9
    assert hb_lib.hb_conv2d_nhwc(*args) == _lib.HB_ERR_SHAPE
    # packed conv: scratch too small
    rc = hb_lib.hb_conv2d_nhwc_packed(p, p, p, 1, 7, 7, 64, 64, 3, 3, 1, 1, 1, 1, 1, 64, p, 16, None, None)
    assert rc == _lib.HB_ERR_SCRATCH
    assert hb_lib.hb_conv2d_packed_scratch_bytes(64, 64, 3, 3) == 3 * 3 * 64 * 64


def test_argument_errors_of_the_neighbour_operators(hb_lib):
    """gemv, scan, the 1-D / 3-D / NCHW convolutions: bad shapes, missing or small scratch and
    misaligned scratch are answered on the host."""
    from heron_b200 import _lib
    buf = np.zeros(1 << 16, dtype=np.uint8)
    base = (buf.ctypes.data + 255) & ~255
    p = ctypes.c_void_p(base)
    F16, F32, U8, S8, S32 = _lib.HB_F16, _lib.HB_F32, _lib.HB_U8, _lib.HB_S8, _lib.HB_S32
    assert hb_lib.hb_gemv(p, p, p, 0, 64, F16, F16, F32, None, None) == _lib.HB_ERR_SHAPE
    assert hb_lib.hb_gemv(p, p, p, 64, 12, U8, S8, S32, None, None) == _lib.HB_ERR_SHAPE  # K bytes % 16
    assert hb_lib.hb_gemv(p, p, p, 64, 64, F16, S8, F32, None, None) == _lib.HB_ERR_DTYPE
    assert hb_lib.hb_scan_scratch_bytes(100, 48, F16) == 100 * 48 * 2
    assert hb_lib.hb_scan_scratch_bytes(100, 48, U8) == 100 * 48
    assert hb_lib.hb_scan(p, p, 16, 100, 48, F16, F32, None, 0, None, None) == _lib.HB_ERR_SCRATCH
    assert hb_lib.hb_scan(p, p, 16, 100, 48, F16, F32, p, 100, None, None) == _lib.HB_ERR_SCRATCH
    assert hb_lib.hb_scan(p, p, 0, 100, 48, F16, F32, p, 1 << 15, None, None) == _lib.HB_ERR_SHAPE
    # NCHW family: window larger than the padded image, no scratch, scratch not 256-byte aligned
    assert hb_lib.hb_conv2d_nchw_scratch_bytes(2, 4, 4, 16, 16, 7, 7, 1, 1, 0, F16, F16) == 0
    need = hb_lib.hb_conv2d_nchw_scratch_bytes(2, 8, 8, 16, 16, 3, 3, 1, 1, 1, F16, F16)
    assert need > 0 and need % 256 == 0
    args = [p, p, p, 2, 8, 8, 16, 16, 3, 3, 1, 1, 1, F16, F16, F16]
    assert hb_lib.hb_conv2d_nchw(*args, None, 0, None, None) == _lib.HB_ERR_SCRATCH
    assert hb_lib.hb_conv2d_nchw(*args, p, need - 1, None, None) == _lib.HB_ERR_SCRATCH
    assert hb_lib.hb_conv2d_nchw(*args, ctypes.c_void_p(base + 16), need, None, None) == _lib.HB_ERR_ALIGN
    assert hb_lib.hb_conv1d_ncw_scratch_bytes(2, 5, 16, 16, 9, 1, 0, F16, F16) == 0
    assert hb_lib.hb_conv1d_ncw(p, p, p, 2, 50, 16, 16, 3, 1, 1, F16, F16, F16, None, 0, None, None) == _lib.HB_ERR_SCRATCH
    assert hb_lib.hb_conv3d_ncdhw_scratch_bytes(1, 2, 4, 4, 16, 16, 3, 3, 3, 1, 1, 1, 0, F16, F16) == 0  # depth 2 < 3 taps
    assert hb_lib.hb_conv3d_ncdhw_scratch_bytes(1, 2, 4, 4, 16, 16, 3, 3, 3, 1, 1, 1, 1, F16, F16) > 0
    rc = hb_lib.hb_conv3d_ncdhw(p, p, p, 1, 2, 4, 4, 16, 16, 3, 3, 3, 1, 1, 1, 1, F16, F16, F16, None, 0, None, None)
    assert rc == _lib.HB_ERR_SCRATCH
    rc = hb_lib.hb_conv1d_nwc_packed(p, p, p, 1, 50, 30, 64, 3, 1, 1, 1, 64, p, 1 << 15, None, None)
    assert rc == _lib.HB_ERR_SHAPE  # CI % 4
    rc = hb_lib.hb_conv1d_nwc_packed(p, p, p, 1, 50, 32, 64, 3, 1, 1, 1, 40, p, 1 << 15, None, None)
    assert rc == _lib.HB_ERR_SHAPE  # sco


def test_no_cpu_fallback(hb_lib):
    """Without a usable sm_100 device a well-formed call reports HB_ERR_DEVICE instead of
    computing anywhere else."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the refusal is what a CPU-only host shows")
    from heron_b200 import _lib
    buf = np.zeros(1 << 16, dtype=np.uint8)
    p = ctypes.c_void_p((buf.ctypes.data + 15) & ~15)
    assert hb_lib.hb_gemm(p, p, p, 64, 64, 64, _lib.HB_U8, _lib.HB_S8, _lib.HB_S32, None, None) == _lib.HB_ERR_DEVICE
    assert hb_lib.hb_sm_count() == -_lib.HB_ERR_DEVICE
    v = ctypes.c_int(0)
    assert hb_lib.hb_last_status(ctypes.byref(v)) == _lib.HB_ERR_DEVICE
    h = ctypes.c_void_p()
    assert hb_lib.hb_plan_gemm(ctypes.byref(h), p, p, p, 64, 64, 64, _lib.HB_U8, _lib.HB_S8, _lib.HB_S32, None) == _lib.HB_ERR_DEVICE
    assert not h.value


def test_front_end_refuses_cpu_tensors(hb_lib):
    import torch
    from heron_b200 import kernels
    a = torch.zeros(64, 64, dtype=torch.uint8)
    b = torch.zeros(64, 64, dtype=torch.int8)
    with pytest.raises(ValueError, match="no CPU path"):
        kernels.gemm(a, b, out=torch.zeros(64, 64, dtype=torch.int32))


def test_library_limits_match_the_constraint_model(hb_lib):
    from heron_b200 import _lib
    from heron_b200.schedule.context import B200_LIMITS
    lim = _lib.kernel_limits()
    for key in ("max_shared_memory_per_block", "tmem_columns", "tile_m", "max_stages", "epilogue_staging_bytes",
                "smem_slack_bytes"):
        assert lim[key] == B200_LIMITS[key], key
    assert lim["static_scratch_bytes"] == hb_lib.hb_conv2d_packed_noalloc_max_bytes()


# ---- the balanced schedule's partition rule (evaluated on the host, no GPU) ----------------------
def _runs(lib, tiles, per_tile, pairs):
    import ctypes
    out = []
    for i in range(pairs):
        a, b = ctypes.c_int(-1), ctypes.c_int(-1)
        assert lib.hb_balanced_run(tiles, per_tile, pairs, i, ctypes.byref(a), ctypes.byref(b)) == 0
        out.append((a.value, b.value))
    return out


def _pieces(run, per_tile):
    """The tiles a run touches, in the order the kernel's roles take them: the run's last tile (if
    the run ends inside it), the run's first tile (if it starts inside it), then the whole tiles."""
    lo, hi = run
    if hi <= lo:
        return []
    t_lo, s_lo = divmod(lo, per_tile)
    t_hi, s_hi = divmod(hi, per_tile)
    out = []
    if s_hi > 0:
        if t_lo == t_hi:
            return [(t_hi, s_lo, s_hi)]
        out.append((t_hi, 0, s_hi))
    if s_lo > 0:
        out.append((t_lo, s_lo, per_tile))
    out.extend((t, 0, per_tile) for t in range(-(-lo // per_tile), t_hi))
    return out


@pytest.mark.parametrize("tiles,per_tile,pairs", [
    (392, 18, 74), (196, 18, 74), (98, 18, 74), (50, 18, 74), (256, 32, 74), (256, 64, 148),
    (1, 40, 8), (75, 4, 74), (74, 9, 74), (1000, 1, 148), (5, 1000, 148), (149, 4, 148)])
def test_balanced_runs_cover_every_stage_once_and_pair_up_their_shared_tiles(hb_lib, tiles, per_tile, pairs):
    # (the library plans this schedule only when every pair gets at least four stages)
    assert tiles * per_tile >= 4 * pairs
    runs = _runs(hb_lib, tiles, per_tile, pairs)
    total = tiles * per_tile
    assert runs[0][0] == 0 and runs[-1][1] == total
    for (a0, a1), (b0, b1) in zip(runs, runs[1:]):
        assert a0 <= a1 == b0 <= b1, "runs are consecutive and in order"
    # the kernel's own walker (compiled for the host) takes the pieces in the order restated above
    import ctypes
    for i, run in enumerate(runs):
        buf = (ctypes.c_int * (3 * 64))()
        n = hb_lib.hb_balanced_pieces(tiles, per_tile, pairs, i, buf, 64)
        want = _pieces(run, per_tile)
        assert n == len(want)
        assert [tuple(buf[3 * j:3 * j + 3]) for j in range(min(n, 64))] == want[:64]
    seen = {}
    for i, run in enumerate(runs):
        for (t, s0, s1) in _pieces(run, per_tile):
            assert 0 <= s0 < s1 <= per_tile and 0 <= t < tiles
            for s in range(s0, s1):
                assert (t, s) not in seen, "stage walked twice"
                seen[(t, s)] = i
    assert len(seen) == total
    # hand-overs: a piece that stops short of its tile's last stage stores partial sums and raises
    # the flags of the NEXT pair, whose run must hold the continuation of the very same tile; a
    # piece that starts inside a tile waits for its own pair's flags, raised by the pair before
    for i, run in enumerate(runs):
        ps = _pieces(run, per_tile)
        producers = [pc for pc in ps if pc[2] < per_tile]
        consumers = [pc for pc in ps if pc[1] > 0]
        assert len(producers) <= 1 and len(consumers) <= 1
        for (t, s0, s1) in producers:
            nxt = [pc for pc in _pieces(runs[i + 1], per_tile) if pc[1] > 0]
            assert nxt == [(t, s1, nxt[0][2])], (i, (t, s0, s1), nxt)
        for (t, s0, s1) in consumers:
            prv = [pc for pc in _pieces(runs[i - 1], per_tile) if pc[2] < per_tile]
            assert prv and prv[0][0] == t and prv[0][2] == s0
        # shared tiles come first: the producer piece, then the consumer piece, then whole tiles
        kinds = ["p" if pc[2] < per_tile else ("c" if pc[1] > 0 else "w") for pc in ps]
        assert kinds == sorted(kinds, key="pcw".index), kinds
    # cuts stay two stages clear of tile edges (or sit on them)
    for a0, _ in runs:
        r = a0 % per_tile
        assert r == 0 or (2 <= r <= per_tile - 2)


def test_balanced_runs_are_level(hb_lib):
    runs = _runs(hb_lib, 50, 18, 74)   # 128 images of the int8 ResNet layer: 50 pair tiles, 74 pairs
    sizes = [b - a for a, b in runs]
    assert max(sizes) <= 900 // 74 + 1 + 2 and min(sizes) >= 900 // 74 - 2


def test_balanced_walker_random_shapes(hb_lib):
    """The kernel's walker over random (tiles, stages per tile, pairs): every stage exactly once,
    at most one piece per run that starts inside a tile and one that ends inside one, shared tiles
    first."""
    import ctypes
    import random
    rnd = random.Random(7)
    for _ in range(300):
        pairs = rnd.choice([1, 2, 3, 37, 74, 148])
        per_tile = rnd.randint(1, 80)
        tiles = rnd.randint(max(1, -(-4 * pairs // per_tile)), max(2, -(-4 * pairs // per_tile)) + rnd.randint(0, 400))
        seen = set()
        buf = (ctypes.c_int * (3 * 512))()
        for i in range(pairs):
            n = hb_lib.hb_balanced_pieces(tiles, per_tile, pairs, i, buf, 512)
            assert 0 <= n <= 512
            kinds = []
            for j in range(n):
                t, s0, s1 = buf[3 * j], buf[3 * j + 1], buf[3 * j + 2]
                assert 0 <= t < tiles and 0 <= s0 < s1 <= per_tile
                for st in range(s0, s1):
                    assert (t, st) not in seen
                    seen.add((t, st))
                kinds.append("p" if s1 < per_tile else ("c" if s0 > 0 else "w"))
            assert kinds.count("p") <= 1 and kinds.count("c") <= 1
            assert kinds == sorted(kinds, key="pcw".index), (tiles, per_tile, pairs, i, kinds)
        assert len(seen) == tiles * per_tile, (tiles, per_tile, pairs)
