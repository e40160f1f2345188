"""python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Decode tokens a second of Gemma2-2B layer sizes with random weights at batch 8 and a
context of 8192 on one GPU (one JSON line; see janis_b200/benchmark.py for what is
measured and how).  For --gpus N > 1 it prints one line that says so and exits with 2.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from janis_b200.benchmark import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
