#!/usr/bin/env python3
"""Benchmark entry point. It measures nothing, and says so.

The benchmark this file is meant to run -- routed tokens/s through threshold
routing, CSR build, row gather, expert-parallel dispatch/combine and weighted
combine -- is defined relative to an implementation in the reference project
bat0001/peer-review-agents. That project holds no such implementation (it is a
pure-Python launcher for LLM reviewing agents: no tensor, Triton, CUDA or
collective code; see tests/test_hot_path_verification.py, which re-checks
this). The specification of this build says to record that and stop rather
than invent a hot path, so no kernel, oracle or CPU baseline exists here.

Both arms therefore print ONE JSON line carrying an "unavailable" reason and a
null value, touch no GPU, and exit 0:

    python bench.py [--gpus N --steps K --warmup W]            # this repository's arm
    python bench.py --impl reference [--gpus N ...]            # the reference's arm

Under torchrun only rank 0 prints; the other ranks exit 0 without work.
"""

import argparse
import json
import os
import sys

METRIC = "routed tokens/s (route+dispatch+combine)"
UNIT = "tokens/s"

WHY_OWN = (
    "hot path absent from the reference (no MoE routing / CSR / permutation / "
    "dispatch-combine code, no API, no golden vectors); build stopped as its "
    "specification directs instead of inventing one - nothing to measure"
)
WHY_REFERENCE = (
    "the reference has no CPU or GPU implementation of this path to time; "
    "it is a pure-Python agent-launcher CLI"
)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("b200", "reference"), default="b200")
    args = ap.parse_args(argv)

    if int(os.environ.get("RANK", "0")) != 0:
        return 0

    if args.impl == "reference":
        line = {"impl": "reference", "unavailable": WHY_REFERENCE, "metric": METRIC,
                "value": None, "unit": UNIT, "n_gpus": args.gpus}
    else:
        line = {
            "metric": METRIC, "value": None, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None,
            "higher_is_better": True, "scaling": None, "vs_baseline": None,
            "dtype": None, "data": "none", "config": {"workload": None},
            "e2e": None, "roofline": None, "cpu_baseline": None, "clocks": None,
            "gpu_launches": 0, "unavailable": WHY_OWN,
        }
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
