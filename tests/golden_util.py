"""Loader of tests/golden/kat.npz (see tests/golden/make_golden.py for what the cases are)."""
import os

import numpy as np

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kat.npz")


def load_cases(name="kat.npz"):
    data = np.load(os.path.join(os.path.dirname(_PATH), name))
    cases = {}
    for key in data.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = data[key]
    for case in cases.values():
        for f in ("stride", "pad", "dil"):
            if f in case:
                case[f] = int(case[f])
    return cases


def run_case(name, case, gemm_int, bmm_int, gemm_f16, conv_int, conv_f16, conv_packed):
    """Dispatches a golden case to an implementation's functions and returns its output."""
    if name.startswith("gemm_f16"):
        return gemm_f16(case["a"], case["b"])
    if name.startswith("gemm"):
        return gemm_int(case["a"], case["b"])
    if name.startswith("bmm"):
        return bmm_int(case["a"], case["b"])
    if name.startswith("conv_packed"):
        return conv_packed(case["x"], case["w"], case["stride"], case["pad"], case["dil"])
    if name.startswith("conv_f16"):
        return conv_f16(case["x"], case["w"], case["stride"], case["pad"], case["dil"], case["out"].dtype)
    return conv_int(case["x"], case["w"], case["stride"], case["pad"], case["dil"])


def assert_matches(name, got, want):
    """Bit-exact for integers; for floating point the largest error within 1e-2 of the largest
    magnitude and every element within 1e-2 |want| + 1e-3 RMS(want) (the benchmark's stated
    relative tolerance with an absolute floor)."""
    assert got.shape == want.shape, name
    if want.dtype.kind in "iu":
        assert got.dtype == want.dtype, name
        assert np.array_equal(got, want), name
    else:
        w64 = want.astype(np.float64)
        diff = np.abs(got.astype(np.float64) - w64)
        scale = max(float(np.abs(w64).max()), 1e-30)
        assert float(diff.max()) / scale <= 1e-2, (name, float(diff.max()) / scale)
        atol = 1e-3 * float(np.sqrt(np.mean(w64 * w64)))
        assert (diff <= 1e-2 * np.abs(w64) + atol).all(), (name, "per-element bound")


def run_neighbour_case(name, case, gemv, conv1d_ncw, conv1d_nwc_packed):
    """The same for tests/golden/kat_neighbours.npz (gemv and the 1-D convolutions)."""
    if name.startswith("gemv"):
        return gemv(case["a"], case["x"])
    if name.startswith("c1d_ncw"):
        return conv1d_ncw(case["x"], case["w"], case["stride"], case["pad"])
    return conv1d_nwc_packed(case["x"], case["w"], case["stride"], case["pad"], case["dil"])
