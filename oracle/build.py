"""Build recipe for the CPU parity checker (test infrastructure, not product code).

Compiles the C++ restatement of the reference's scalar path into ``oracle/liboracle.so``.
``-O2 -ffp-contract=off`` mirrors the reference's optimised test profile without letting the
compiler fuse multiply-adds, so every product and sum rounds where the reference's does.

The reference itself is Rust; no Rust toolchain exists in this environment, so there is no
``oracle/_ref`` build of the reference's own sources.
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["models.cpp"]
HEADERS = ["scalar.h"]
OUTPUT = os.path.join(HERE, "liboracle.so")


def needs_build() -> bool:
    if not os.path.exists(OUTPUT):
        return True
    built = os.path.getmtime(OUTPUT)
    return any(os.path.getmtime(os.path.join(HERE, f)) > built for f in SOURCES + HEADERS)


def build(force: bool = False) -> str:
    if not force and not needs_build():
        return OUTPUT
    cmd = [
        "g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC", "-shared",
        "-o", OUTPUT,
    ] + [os.path.join(HERE, s) for s in SOURCES]
    subprocess.run(cmd, check=True)
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
