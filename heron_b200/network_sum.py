"""Whole-network operator sums: the reference's figure-10 experiment
(tests/figure10/run.py, tests/figure10/configs/{resnet50,vgg16,inceptionv3,bert}.json) on the B200
kernels.

    python -m heron_b200.network_sum -c heron_b200/configs/resnet50_nchw_fp16.json [--tune N]

Every case of the JSON file is ``[op, shape arguments, count]``: the operator is instantiated
(library default knobs, or the best of an ``N``-trial CGA run with ``--tune N``), timed on the
device with CUDA events, and the network figure is sum(latency * count) — the quantity the
reference's PyTorch baselines log (tests/figure10/pytorch/logs/*.log).  The layer tables are the
published ResNet-50 / VGG-16 / Inception-v3 / BERT-base operator shapes at batch 16, in the
reference's case format.
"""
import argparse
import json
import os

from .config import Config, configFromFile
from .environment import Env
from .ops import cuda as heron_cuda
from .runner import LocalRunner, measure_handle, measure_option, reduce_costs
from .task import Task


def time_case(name, op_name, case, in_dtype, out_dtype, tune, number, repeat, out_name):
    cfg = Config()
    cfg.codegen_type = "GPU_TENSOR_CORE"
    cfg.out_name, cfg.opt_method, cfg.max_trials, cfg.parallel = out_name, "CGA", tune, False
    cfg.measure_time_per_round, cfg.pop_num, cfg.select_num, cfg.iter_walks = 16, 64, 32, 3
    params = list(case) + [in_dtype, out_dtype]
    if tune > 0:
        env = Env(measure_option(runner=LocalRunner(number=number, repeat=repeat)), cfg)
        task = env.createTask(name, heron_cuda.getOpFromName(op_name), params, "cuda")
        env.tune(name)
        handle, args = task.apply_best(os.path.join(cfg.log_dir, "records.txt"))
    else:
        task = Task(name, heron_cuda.getOpFromName(op_name), params, "cuda")
        cfg.log_dir = None
        task.config = cfg
        outs = task.getOut()
        from .task import KernelHandle
        handle, args = KernelHandle(outs[0].op, {}), outs[0].op.input_tensors + outs
    res = measure_handle(task, handle, args, number=number, repeat=repeat, min_repeat_ms=20)
    if res.error_no != 0:
        raise RuntimeError("%s failed: %s" % (name, res))
    return reduce_costs(list(res.costs)), handle.knobs


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-c", "--config", required=True)
    ap.add_argument("--tune", type=int, default=0, help="CGA trials per layer (0: library defaults)")
    ap.add_argument("--json", default="", help="write per-layer results here")
    args = ap.parse_args(argv)
    config = configFromFile(args.config)
    rows, total = [], 0.0
    for name, entry in config.cases.items():
        op_name, case = entry[0], entry[1]
        count = entry[2] if len(entry) > 2 else 1
        sec, knobs = time_case(name.strip(), op_name, case, config.in_dtype, config.out_dtype, args.tune,
                               config.runner_number, config.runner_repeat, config.out_name)
        total += sec * count
        rows.append({"layer": name.strip(), "op": op_name, "case": case, "count": count, "latency_ms": sec * 1e3,
                     "knobs": knobs})
        print("%-10s %-5s %-44s x%-2d %9.4f ms" % (name.strip(), op_name, case, count, sec * 1e3), flush=True)
    print("network sum: %.4f ms" % (total * 1e3))
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"config": args.config, "tune": args.tune, "sum_ms": total * 1e3, "layers": rows}, f, indent=1)
    return total


if __name__ == "__main__":
    main()
