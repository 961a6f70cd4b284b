"""Builds the CPU oracle (test infrastructure only) into oracle/liboracle_sampler.so.

Run as `python -m oracle.build`, or call `build()`; the root build entry calls
it too. -ffp-contract=off and no fast-math: every f32 operation of the
reference must stay one rounded operation, in source order.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(HERE, "sampler_oracle.cpp")
LIBRARY = os.path.join(HERE, "liboracle_sampler.so")

FLAGS = ["-std=c++17", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-pthread",
         "-Wall", "-Wextra"]


def is_stale() -> bool:
    return (not os.path.exists(LIBRARY)) or os.path.getmtime(LIBRARY) < os.path.getmtime(SOURCE)


def build(force: bool = False) -> str:
    if force or is_stale():
        cmd = ["g++", *FLAGS, SOURCE, "-o", LIBRARY]
        subprocess.run(cmd, check=True)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
