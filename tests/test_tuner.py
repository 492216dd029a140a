"""The search stack on CPU: CGA / CRAND / SA over the kernels' knob space with a synthetic
measurement function standing in for the device, records.txt / stat.txt formats, warm start."""
import json
import math
import os
import random

import numpy as np
import pytest

from heron_b200.config import Config
from heron_b200.environment import Env
from heron_b200.ops import cuda as heron_cuda
from heron_b200.perf.perfBuffer import perfBuffer, warm_start
from heron_b200.runner import MeasureErrorNo, MeasureResult, measure_option
from heron_b200.utils import genKey


def fake_measure(task, handle, args):
    """A smooth synthetic cost: wide tiles and deep rings are fast, one knob combination fails."""
    k = handle.knobs
    if k["tile_n"] == 32 and k["stages"] == 1:
        return MeasureResult((RuntimeError("injected failure"),), MeasureErrorNo.RUNTIME_DEVICE, 0.0, 0.0)
    t = 1e-4 * (1.0 + 256.0 / k["tile_n"]) * (1.0 + 2.0 / k["stages"]) * (1.2 if k["swizzle_bytes"] < 128 else 1.0)
    t *= 0.8 if k["cta_group"] == 2 else 1.0
    return MeasureResult((t,), MeasureErrorNo.NO_ERROR, 0.0, 0.0)


def make_env(tmp_path, method, trials=48):
    cfg = Config()
    cfg.out_name = str(tmp_path)
    cfg.opt_method = method
    cfg.max_trials = trials
    cfg.measure_time_per_round = 16
    cfg.pop_num = 40
    cfg.select_num = 20
    cfg.iter_walks = 2
    cfg.parallel = False
    cfg.codegen_type = "GPU_TENSOR_CORE"
    env = Env(measure_option(), cfg, measure_fn=fake_measure)
    env.createTask("G2", heron_cuda.getOpFromName("gemm"), [4096, 4096, 4096, "float16", "float32"], "cuda")
    return env


@pytest.mark.parametrize("method", ["CGA", "CRAND", "SA", "GA", "SDGA", "SRGA", "IDEA"])
def test_tuning_loop_improves_and_writes_records(tmp_path, method):
    random.seed(7)
    np.random.seed(7)
    env = make_env(tmp_path, method)
    env.tune("G2")
    log_dir = env.config.log_dir
    rows = [json.loads(r) for r in open(os.path.join(log_dir, "records.txt"))]
    assert 16 <= len(rows) <= 48
    for r in rows:
        assert set(r) == {"code", "perf", "latency", "time", "param"}
        if r["perf"] != 0:
            assert math.isclose(r["latency"], math.exp(-r["perf"]), rel_tol=1e-9)
    assert len({r["code"] for r in rows}) == len(rows)  # no candidate measured twice
    stat = [l.strip().split(",") for l in open(os.path.join(log_dir, "stat.txt"))]
    assert len(stat) == math.ceil(48 / 16) + 1 and all(len(s) == 6 for s in stat)
    assert os.path.exists(os.path.join(log_dir, "schedule.py"))
    assert os.path.exists(os.path.join(log_dir, "constraints.py"))
    best = max(r["perf"] for r in rows)
    # the synthetic optimum is tile_n=256, 12.. stages as deep as fits, cta_group 2: ln(1/t) ~ 8.6
    assert best > 8.2
    handle, _ = env.task.apply_best(os.path.join(log_dir, "records.txt"))
    assert handle.knobs["tile_n"] >= 192


def test_failed_candidates_score_zero_and_are_not_training_data(tmp_path):
    env = make_env(tmp_path, "CRAND")
    env.init_dir()
    env.task.make_stage_schedules()
    from heron_b200.sample import Sample
    s = Sample(env.task)
    km = s.knob_manager
    known = {genKey("P", "dense", "n", param_name="tile_n"): [32], genKey("P", "dense", "k", param_name="stages"): [1]}
    valid, point = km.randSample(known)
    s.set_point(point, valid)
    env.evalSamples([s])
    assert s.perf == 0.0 and not s.valid
    assert env.perf_buffer.data_y == [] and env.perf_buffer.perfs[s.stmt_code] == 0.0


def test_warm_start_reloads_records(tmp_path):
    random.seed(1)
    np.random.seed(1)
    env = make_env(tmp_path, "CRAND", trials=16)
    env.tune("G2")
    path = os.path.join(env.config.log_dir, "records.txt")
    fresh = perfBuffer(Config())
    n = warm_start(fresh, env.task, path)
    assert n == len(env.perf_buffer.perfs)
    assert fresh.best_perf == env.perf_buffer.best_perf
    assert sorted(fresh.data_y) == sorted(env.perf_buffer.data_y)


def test_cost_model_learns_the_synthetic_cost(tmp_path):
    random.seed(3)
    np.random.seed(3)
    env = make_env(tmp_path, "CRAND", trials=64)
    env.tune("G2")
    model = env.tuner.cost_model
    assert model.bst is not None
    samples = env.perf_buffer.samples
    pred = model.predict(samples)
    truth = np.array([s.perf for s in samples])
    assert np.corrcoef(pred, truth)[0, 1] > 0.9
    assert model.bst.get_score()  # feature weights, as the key-variable ranking expects
