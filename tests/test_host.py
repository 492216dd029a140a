"""Host-side mirror of the reference interface: operator registry, Task, knob space and its
solver, configuration, partitioning — all on CPU."""
import json
import os
import random

import numpy as np
import pytest

from heron_b200.config import Config, configFromFile
from heron_b200.multi import Job, partition, shard_case
from heron_b200.ops import cuda as heron_cuda, x86 as heron_cpu
from heron_b200.schedule.constraints import EQ, LE, KnobManager, ProdTwo, Solver, Sum
from heron_b200.task import Task
from heron_b200.utils import Code, DeCode, genKey


class _Ctx:
    def __init__(self):
        self.info = None
        self.axis_map = None

    def set_info(self, info):
        self.info = info

    def set_axis_map(self, m):
        self.axis_map = m


def test_registry_names_and_signatures():
    assert heron_cuda.getOpFromName("gemm").__name__ == "heron_dense"
    assert heron_cuda.getOpFromName("bmm").__name__ == "heron_batch_matmul"
    assert heron_cuda.getOpFromName("c2d_nhwc").__name__ == "heron_conv2d_nhwc_tensorcore"
    assert heron_cpu.getOpFromName("c2d").__name__ == "heron_conv2d_nhwc"
    assert heron_cuda.getOpFromName("c2d").__name__ == "heron_conv2d_nchw_tensorcore"
    assert heron_cuda.getOpFromName("dil").__name__ == "heron_dil_tensorcore"
    assert heron_cpu.getOpFromName("dil").__name__ == "heron_dil_nhwc"
    assert heron_cuda.getOpFromName("gemv").__name__ == "heron_gemv"
    assert heron_cpu.getOpFromName("gemv").__name__ == "heron_gemv"
    assert heron_cuda.getOpFromName("c1d").__name__ == "heron_conv1d_ncw_tensorcore"
    assert heron_cuda.getOpFromName("scan").__name__ == "heron_scan"
    assert heron_cpu.getOpFromName("scan").__name__ == "heron_scan"
    assert heron_cpu.getOpFromName("c1d").__name__ == "heron_conv1d_nwc"
    assert heron_cuda.getOpFromName("t2d").__name__ == "heron_conv2d_nchw_transposed_tensorcore"
    assert heron_cpu.getOpFromName("t2d").__name__ == "heron_conv2d_transposed_nhwc"
    assert heron_cuda.getOpFromName("c3d").__name__ == "heron_conv3d_ncdhw_tensorcore"
    with pytest.raises(NotImplementedError):
        heron_cuda.getOpFromName("dep")
    with pytest.raises(NotImplementedError):
        heron_cpu.getOpFromName("c3d")
    with pytest.raises(KeyError):
        heron_cuda.getOpFromName("nonsense")


def test_t2d_refuses_the_strides_the_reference_leaves_undefined():
    ctx = _Ctx()
    (out,) = heron_cuda.getOpFromName("t2d")(ctx, 16, 56, 56, 64, 64, 3, 3, 1, 1, 1, 0, "float16", "float16")
    assert out.shape == (16, 64, 56, 56) and out.op.params["padding"] == 1
    (out,) = heron_cuda.getOpFromName("t2d")(ctx, 16, 14, 14, 256, 512, 3, 3, 1, 0, 1, 0, "float16", "float16")
    assert out.shape == (16, 512, 16, 16) and out.op.params["padding"] == 2
    with pytest.raises(NotImplementedError):
        heron_cuda.getOpFromName("t2d")(ctx, 16, 56, 56, 64, 128, 1, 1, 2, 0, 1, 0, "float16", "float16")
    with pytest.raises(NotImplementedError):
        heron_cpu.getOpFromName("t2d")(ctx, 1, 56, 56, 64, 128, 1, 1, 2, 0, 1, 0, "OhwI64o4i", "uint8", "int32")
    (out,) = heron_cpu.getOpFromName("t2d")(ctx, 1, 14, 14, 64, 64, 3, 3, 1, 1, 2, 0, "OhwI64o4i", "uint8", "int32")
    assert out.op.params["padding"] == 3 and out.shape == (1, 16, 16, 1, 64)


def test_gemm_op_layout_and_hints():
    ctx = _Ctx()
    (out,) = heron_cuda.getOpFromName("gemm")(ctx, 128, 64, 32, "float16", "float32")
    a, b = out.op.input_tensors
    assert a.shape == (128, 64) and b.shape == (32, 64) and out.shape == (128, 32)  # B is (N, K)
    assert out.dtype == "float32" and a.name == "A" and b.name == "B" and out.op.name == "dense"
    assert ctx.info["name"] == "tensorcore" and ctx.info["loadB"][2] == "col_major"
    assert "dense.wmma.accumulator" in ctx.axis_map


def test_x86_ops_ignore_dtype_arguments():
    ctx = _Ctx()
    (out,) = heron_cpu.getOpFromName("gemm")(ctx, 64, 64, 64, "float16", "float16")
    a, b = out.op.input_tensors
    assert (a.dtype, b.dtype, out.dtype) == ("uint8", "int8", "int32")
    assert ctx.info["name"] == "x86_dot"


def test_bmm_requires_batch_gt_one():
    with pytest.raises(AssertionError):
        heron_cuda.getOpFromName("bmm")(_Ctx(), 1, 64, 64, 64, "int8", "int32")


def test_conv_shapes_and_shape_rule():
    ctx = _Ctx()
    (out,) = heron_cuda.getOpFromName("c2d_nhwc")(ctx, 32, 56, 56, 64, 64, 3, 3, 1, 1, 1, "float16", "float16")
    x, w = out.op.input_tensors
    assert x.shape == (32, 56, 56, 64) and w.shape == (3, 3, 64, 64) and out.shape == (32, 56, 56, 64)
    (out,) = heron_cuda.getOpFromName("c2d_nhwc")(_Ctx(), 16, 14, 14, 256, 512, 3, 3, 2, 1, 1, "float16", "float16")
    assert out.shape == (16, 7, 7, 512)
    with pytest.raises(AssertionError):
        heron_cuda.getOpFromName("c2d_nhwc")(_Ctx(), 3, 8, 8, 16, 16, 3, 3, 1, 1, 1, "float16", "float16")


def test_x86_conv_packed_shapes():
    (out,) = heron_cpu.getOpFromName("c2d")(_Ctx(), 1024, 7, 7, 512, 512, 3, 3, 1, 1, 1, "OhwI64o4i", "uint8", "int32")
    x, w = out.op.input_tensors
    assert w.shape == (8, 3, 3, 128, 64, 4) and out.shape == (1024, 7, 7, 8, 64)
    with pytest.raises(AssertionError):
        heron_cpu.getOpFromName("c2d")(_Ctx(), 1, 7, 7, 64, 64, 3, 3, 1, 1, 1, "OhwI16o4i", "uint8", "int32")


def test_genkey_and_code():
    assert genKey("L", "dense", "i") == "L#ST:dense,AX:i"
    assert genKey("P", "dense", "n", param_name="tile_n") == "P#ST:dense,AX:n,PA:tile_n"
    assert genKey("V", "dense", "k", var_name="x") == "V#ST:dense,AX:k,VA:x"
    assert DeCode(Code([3, 14, 15])) == [3, 14, 15]


def test_solver_products_sums_conditions():
    s = Solver()
    for name, lo, hi in [("a", 1, 64), ("b", 1, 64), ("m", 0, 100000), ("x", 0, 300), ("c0", 0, 1), ("c1", 0, 1)]:
        s.addVal(name, lo, hi, lo)
    s.primitives += [ProdTwo([64, ["a", "b"]]), ProdTwo(["m", ["a", "x"]]), LE(["m", 2000]),
                     EQ(["x", 128], cond="c0"), EQ(["x", 256], cond="c1"), Sum([1, ["c0", "c1"]])]
    random.seed(0)
    seen = set()
    for _ in range(30):
        ok, point = s.solve({}, {})
        assert ok
        vals = dict(zip(s.vals.keys(), point))
        assert s.SATScore(vals) == 0
        assert vals["a"] * vals["b"] == 64 and vals["m"] == vals["a"] * vals["x"] <= 2000
        seen.add((vals["a"], vals["x"]))
    assert len(seen) >= 3
    assert s.validate({"a": 8, "x": 256}) == (False, None)
    ok, point = s.validate({"a": 4, "x": 256})
    assert ok and dict(zip(s.vals.keys(), point))["m"] == 1024
    ok, point = s.solve({}, {"a": [2, 32]})
    assert ok and dict(zip(s.vals.keys(), point))["a"] == 2  # 32 * x > 2000 for either x
    scores, valid = s.MultiSATScore({"a": 8, "b": 8, "m": 2048, "x": 256, "c0": 0, "c1": 1})
    assert not valid and sum(scores) == 48


def _task(op, args, codegen="GPU_TENSOR_CORE", registry=heron_cuda):
    t = Task("T", registry.getOpFromName(op), args, "cuda")
    cfg = Config()
    cfg.codegen_type = codegen
    cfg.log_dir = None
    t.config = cfg
    t.make_stage_schedules()
    return t


def test_task_knob_space_and_instantiate(hb_lib):
    """Every sampled point satisfies the kernel's own knob check (hb_check_knobs)."""
    import ctypes
    from heron_b200 import _lib
    t = _task("gemm", [4096, 4096, 4096, "float16", "float32"])
    km = t.knob_manager
    assert not km.is_building and len(km.knob_names) == 11
    random.seed(3)
    distinct = set()
    for _ in range(40):
        valid, point = km.randSample()
        assert valid and len(point) == len(km.solver.vals)
        handle, args = t.instantiate(km)
        assert [a.name for a in args] == ["A", "B", "dense"]
        k = _lib.HbKnobs.from_dict(handle.knobs)
        smem = ctypes.c_int(0)
        rc = hb_lib.hb_check_knobs(0, 1, 4096, 4096, 4096, 4096, _lib.HB_F16, _lib.HB_F32, ctypes.byref(k),
                                   ctypes.byref(smem), None)
        assert rc == 0, handle.knobs
        assert smem.value == km.solved_knob_vals_phenotype[genKey("V", "dense", "k", var_name="shared_mem_size")]
        distinct.add(tuple(sorted(handle.knobs.items())))
    assert len(distinct) > 10


def test_conv_knob_space_respects_channel_bytes(hb_lib):
    import ctypes
    from heron_b200 import _lib
    t = _task("c2d_nhwc", [16, 9, 9, 16, 64, 3, 3, 1, 1, 1, "float16", "float32"])
    km = t.knob_manager
    random.seed(4)
    for _ in range(20):
        km.randSample()
        handle, _ = t.instantiate(km)
        assert handle.knobs["swizzle_bytes"] == 32  # 16 fp16 channels = 32 bytes
        k = _lib.HbKnobs.from_dict(handle.knobs)
        assert hb_lib.hb_check_knobs(2, 1, 16 * 81, 64, 144, 16, _lib.HB_F16, _lib.HB_F32, ctypes.byref(k), None, None) == 0


def test_conv_algorithm_candidates_follow_the_feasibility_rules():
    """The constraint model offers a conv algorithm only where its rule holds: the fused-row form is
    a subset of the strip kernel's space (same strips plus 12 KiB of exchange), needs fp16, 64
    output channels, a three-tap undilated filter row; a task's candidate list is what the rules say."""
    from heron_b200.schedule.context.context import B200_LIMITS
    from heron_b200.schedule.sched_op import strip_applies, strip_fused_applies, strip_wide_applies
    rnd = random.Random(5)
    seen_fused = 0
    for _ in range(400):
        g = dict(stride=(rnd.choice([1, 1, 2]),) * 2, dilation=(rnd.randint(1, 2), rnd.choice([1, 1, 2])),
                 CI=rnd.choice([64, 128]), CO=rnd.choice([64, 128]), KH=rnd.randint(1, 3), KW=rnd.randint(1, 3),
                 padding=rnd.randint(0, 2), H=rnd.randint(1, 60), W=rnd.randint(1, 140), in_dtype="float16")
        eo = rnd.choice([2, 4])
        fused = strip_fused_applies(g, 2, eo, B200_LIMITS)
        if fused:
            seen_fused += 1
            assert strip_applies(g, 2, eo, B200_LIMITS)
            assert g["CO"] == 64 and g["KW"] == 3 and g["dilation"][1] == 1 and g["stride"] == (1, 1)
            assert g["W"] + 2 * g["padding"] <= 128
    assert seen_fused > 10
    assert not strip_fused_applies(dict(stride=(1, 1), dilation=(1, 1), CI=64, CO=64, KH=3, KW=3, padding=1, H=8, W=8,
                                        in_dtype="uint8"), 1, 4, B200_LIMITS)
    t = _task("c2d_nhwc", [16, 20, 20, 64, 64, 3, 3, 1, 1, 1, "float16", "float16"])
    name = [k for k in t.knob_manager.knob_names if "conv_algo" in k][0]
    assert sorted(t.knob_manager.get_knob_candidates(name)) == [1, 2, 3, 4]
    t = _task("c2d_nhwc", [16, 20, 20, 64, 128, 3, 3, 1, 1, 1, "float16", "float16"])
    name = [k for k in t.knob_manager.knob_names if "conv_algo" in k][0]
    assert 4 not in t.knob_manager.get_knob_candidates(name)
    assert strip_wide_applies(dict(stride=(1, 1), dilation=(1, 1), CI=64, CO=128, KH=3, KW=3, padding=1, H=20, W=20,
                                   in_dtype="float16"), 2, 2, B200_LIMITS)


def test_nchw_first_layer_knob_space_is_the_row_packed_form(hb_lib):
    """3 input channels, 7x7 filter: the library reads a whole filter row (8 taps of 16 bytes) as one
    128-byte K block, and the tuner's space must offer that block size, not the 32 bytes of the
    channel-padded form."""
    t = _task("c2d", [16, 224, 224, 3, 64, 7, 7, 2, 3, 1, "float16", "float16"])
    spans = set()
    random.seed(6)
    for _ in range(30):
        t.knob_manager.randSample()
        handle, _ = t.instantiate(t.knob_manager)
        spans.add(handle.knobs["swizzle_bytes"])
    assert 128 in spans
    t = _task("c2d", [16, 56, 56, 3, 64, 3, 3, 1, 1, 1, "float16", "float16"])
    t.knob_manager.randSample()
    handle, _ = t.instantiate(t.knob_manager)
    assert handle.knobs["swizzle_bytes"] in (32, 64)  # 4 taps of 16 bytes


def test_cga_crossover_keeps_parent_values():
    import copy
    t = _task("bmm", [192, 512, 64, 512, "int8", "int32"])
    random.seed(5)
    m1, m2 = copy.deepcopy(t.knob_manager), copy.deepcopy(t.knob_manager)
    m1.randSample()
    m2.randSample()
    child = copy.deepcopy(t.knob_manager)
    keys = [genKey("P", "batch_matmul", "n", param_name="tile_n"), genKey("P", "batch_matmul", "k", param_name="stages"),
            genKey("P", "batch_matmul", "m", param_name="raster")]
    res, valid = child.constrained_crossover_and_mutate(m1, m2, keys)
    assert valid
    inherited = sum(child.solved_knob_vals_phenotype[k] in (m1.solved_knob_vals_genotype[k], m2.solved_knob_vals_genotype[k])
                    for k in keys)
    assert inherited >= len(keys) - 1
    assert child.solver.SATScore(child.solved_knob_vals_phenotype) == 0


def test_apply_best_reads_records(tmp_path):
    t = _task("gemm", [64, 64, 64, "uint8", "int32"], "CPU", heron_cpu)
    km = t.knob_manager
    random.seed(6)
    rows = []
    for perf in (10.5, 12.9, 11.0):
        km.randSample()
        rows.append(dict(code="c%s" % perf, perf=perf, latency=float(np.exp(-perf)), time=0.0,
                         param=dict(km.solved_knob_vals_phenotype)))
    path = tmp_path / "records.txt"
    path.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    t2 = Task("T", heron_cpu.getOpFromName("gemm"), [64, 64, 64, "uint8", "int32"], "llvm")
    cfg = Config()
    cfg.codegen_type = "CPU"
    cfg.log_dir = None
    t2.config = cfg
    handle, args = t2.apply_best(str(path))
    assert t2.knob_manager.runtime_perf == 12.9
    best = rows[1]["param"]
    assert handle.knobs["tile_n"] == best[genKey("P", "dense", "n", param_name="tile_n")]
    assert [a.dtype for a in args] == ["uint8", "int8", "int32"]


def test_config_from_file(tmp_path):
    ref_style = {"config": {"out_name": "OPS/GEMM", "method": "CGA", "max_trials": 32, "runner_number": 3,
                            "runner_repeat": 4, "runner_timeout": 50, "build_timeout": 50, "in_dtype": "int8",
                            "out_dtype": "int32", "cases": {"G1": ["gemm", [64, 64, 64]]}}}
    p = tmp_path / "quick_start.json"
    p.write_text(json.dumps(ref_style))
    c = configFromFile(str(p))
    assert c.opt_method == "CGA" and c.cases["G1"] == ["gemm", [64, 64, 64]] and c.pop_num == 200
    assert c.crossover_key_ratio == 0.2 and c.measure_time_per_round == 32


def test_partition_and_shard_case():
    assert partition(192, 8) == [(i * 24, 24) for i in range(8)]
    assert partition(10, 4) == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert partition(2, 4) == [(0, 1), (1, 1), (2, 0), (2, 0)]
    for extent, world in [(192, 8), (1024, 4), (7, 3)]:
        parts = partition(extent, world)
        assert sum(c for _, c in parts) == extent
        assert all(parts[i][0] + parts[i][1] == parts[i + 1][0] for i in range(world - 1))
    args, (start, count) = shard_case("c2d_nhwc", [1024, 7, 7, 512, 512, 3, 3, 1, 1, 1], 3, 8)
    assert args[0] == 128 and (start, count) == (384, 128)
    with pytest.raises(ValueError):
        shard_case("gemm", [64, 64, 64], 0, 2)
    args, (start, count) = shard_case("c3d", [8, 8, 56, 56, 64, 64, 3, 3, 3, 1, 1, 1], 1, 4)
    assert args[0] == 2 and (start, count) == (2, 2) and args[1:] == [8, 56, 56, 64, 64, 3, 3, 3, 1, 1, 1]


def _square(x):
    return x * x


def _sleep_forever():
    import time
    time.sleep(60)
    return 1


def test_job_returns_and_times_out():
    j = Job(_square, None, timeout=10)
    j.start((7,))
    assert j.get() == 49
    j = Job(_sleep_forever, None, timeout=0.5)
    j.start(())
    assert j.get() == 0  # the reference's convention for a timed-out worker (multi.py:21-25)
