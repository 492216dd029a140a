"""Command-line driver with the reference's flags (tests/quick_start/dlboost/run.py:68-109):

    python -m heron_b200.run -p {tensorcore,dlboost} -c CONFIG.json [-t records.txt] [-d DEV] [-m TRIALS]

For every case of the JSON file: build the task, tune it (unless ``-t`` names tuned records),
re-apply the best record, time the resulting kernel and print its latency.  Like the reference's
driver it prints PASS when the tuned kernel ran; unlike it, the latency is a CUDA-event median on
the device rather than a TVM ``time_evaluator`` mean.
"""
import argparse
import os

from .config import configFromFile
from .environment import Env
from .ops import cuda as heron_cuda, x86 as heron_cpu
from .runner import LocalRunner, measure_handle, measure_option, reduce_costs


def makeConfig(args):
    config = configFromFile(args.config)
    if args.platform == "tensorcore":
        config.target_name = "cuda"
        config.codegen_type = "GPU_TENSOR_CORE"
        config.get_op = heron_cuda.getOpFromName
    else:
        # the DL Boost operators (uint8 x int8 -> int32, x86 layouts) run on the B200 int8 path
        config.target_name = "cuda -model=b200 (x86 operator semantics)"
        config.codegen_type = "CPU"
        config.get_op = heron_cpu.getOpFromName
    return config


def run(op_name, task_name, params, env):
    config = env.config
    op = config.get_op(op_name)
    task = env.createTask(task_name, op, params, config.target_name)
    task.device_id = config.device_id
    if config.tuned == "":
        env.tune(task_name)
        config.tuned = os.path.join(config.log_dir, "records.txt")
    handle, args = task.apply_best(config.tuned)
    res = measure_handle(task, handle, args, number=config.runner_number, repeat=config.runner_repeat,
                         min_repeat_ms=50, flush_l2=False, device_id=config.device_id)
    if res.error_no != 0:
        print("FAIL", res)
        return 0.0, handle.knobs
    latency = reduce_costs(list(res.costs)) * 1e3
    if latency > 0:
        print("PASS")
    return latency, handle.knobs


def main(argv=None):
    parser = argparse.ArgumentParser(description="Run cases in heron_b200.")
    parser.add_argument("-p", "--platform", choices=["tensorcore", "dlboost"], type=str, default="dlboost")
    parser.add_argument("-c", "--config", type=str, required=True)
    parser.add_argument("-t", "--tuned", type=str, default="")
    parser.add_argument("-d", "--device_id", type=int, default=0)
    parser.add_argument("-sid", "--start_id", type=int, default=0)
    parser.add_argument("-eid", "--end_id", type=int, default=10000)
    parser.add_argument("-v", "--verbose", action="store_true")
    parser.add_argument("-m", "--max-trials", type=int, default=1000000)
    parser.add_argument("--sequential", action="store_true", help="sample in-process instead of forked workers")
    args = parser.parse_args(argv)

    cases = []
    base = makeConfig(args)
    keys = list(base.cases.keys())
    for i in range(args.start_id, min(args.end_id + 1, len(keys))):
        config = makeConfig(args)
        config.max_trials = min(args.max_trials, config.max_trials)
        config.device_id = args.device_id
        config.tuned = args.tuned if i == 0 else ""
        config.verbose = args.verbose
        config.parallel = not args.sequential
        runner = LocalRunner(number=config.runner_number, repeat=config.runner_repeat, min_repeat_ms=0,
                             timeout=config.runner_timeout, device_id=args.device_id)
        op_name, case = config.cases[keys[i]]
        env = Env(measure_option(runner=runner), config)
        latency, knobs = run(op_name, keys[i], case + [config.in_dtype, config.out_dtype], env)
        cases.append((keys[i], case, latency, knobs, env.perf_buffer.best_perf))
    for name, case, latency, knobs, best in cases:
        print("Case %s %s, latency %f ms, knobs %s" % (name, str(case), latency, knobs))
    return cases


if __name__ == "__main__":
    main()
