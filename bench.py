#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5 layer sizes, random weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--model 7b|14b|32b]
                    [--workload decode|mix] [--layers L] [--profile]

Prints ONE JSON line; what it measures and how is written at the top of tensorline_b200/benchmark.py, which holds
the measurements (the `tensorline bench` command runs the same code).  Default: Qwen2.5-7B layer sizes, decode at
batch 8 and a context of 4,096 tokens, with end-to-end, prefill, roofline and batch 1 / 64 figures on the same line.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from tensorline_b200.benchmark import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
