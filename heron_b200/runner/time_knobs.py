"""Device time of one benchmark configuration under explicit knob sets.

    python -m heron_b200.runner.time_knobs --workload cfg5_conv_u8s8_resnet_s4 [--units 128] \
        [--iters 300] [--warm] "balance=1" "balance=2" "balance=2,max_ctas=100" ...

Each positional argument is one knob set (`name=value` pairs separated by commas; an empty string
is the library default).  For every set the operator is planned on rotating buffer sets (more
than the 126 MB L2 between reuses, or one set with --warm), launched `iters` times back to back
and timed with CUDA events; the best of three repetitions is printed with the resolved knobs.
`--units` shrinks the sharded leading dimension (images / batches), e.g. to one rank's shard.
Diagnostic `probe` values only act in a library built with HB_PROBES=1.
"""
import argparse
import json

import numpy as np


def main():
    import torch
    from heron_b200 import _lib, kernels as K
    from heron_b200.workloads import CONFIGS, make_inputs

    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", required=True, choices=sorted(CONFIGS))
    ap.add_argument("--units", type=int, default=None)
    ap.add_argument("--iters", type=int, default=300)
    ap.add_argument("--warm", action="store_true", help="one buffer set: inputs stay in L2")
    ap.add_argument("knobs", nargs="*", default=[""])
    args = ap.parse_args()

    cfg = CONFIGS[args.workload]
    dev = torch.device("cuda", 0)
    shard = (0, args.units) if (args.units and cfg["op"] != "gemm") else None
    host = make_inputs(args.workload, shard=shard) if shard else make_inputs(args.workload)
    out_dtype = K.TORCH_DTYPES[cfg["out_dtype"]]
    nbytes = sum(h.nbytes for h in host)
    n_sets = 1 if args.warm else max(2, min(16, int(np.ceil(300e6 / max(nbytes * 3, 1))) + 1))
    sets = [[torch.from_numpy(np.ascontiguousarray(h)).to(dev) for h in host] for _ in range(n_sets)]

    def plan(ins, knobs):
        if cfg["op"] == "gemm":
            return K.plan_gemm(ins[0], ins[1], out_dtype=out_dtype, knobs=knobs)
        if cfg["op"] == "bmm":
            return K.plan_bmm(ins[0], ins[1], out_dtype=out_dtype, knobs=knobs)
        c = cfg["case"]
        return K.plan_conv2d_nhwc(ins[0], ins[1], c[7], c[8], c[9], out_dtype=out_dtype, knobs=knobs)

    for spec in args.knobs:
        knobs = {kv.split("=")[0].strip(): int(kv.split("=")[1]) for kv in spec.split(",") if kv.strip()}
        try:
            plans = [plan(s, knobs or None) for s in sets]
        except _lib.HeronB200Error as e:
            print(json.dumps({"knobs": knobs, "error": str(e)}))
            continue
        for i in range(20):
            plans[i % n_sets].launch()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.iters):
                plans[i % n_sets].launch()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / args.iters * 1e3)
        status = _lib.last_status()
        print(json.dumps({"workload": args.workload, "units": args.units, "knobs": knobs, "us_per_launch": round(best, 2),
                          "buffer_sets": n_sets, "status": status, "resolved": plans[0].knobs()}), flush=True)
        del plans


if __name__ == "__main__":
    main()
