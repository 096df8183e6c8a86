"""Build ``libbobcat_cuda.so`` in-tree with nvcc for sm_100a.

``python -m bobcat_b200.build`` compiles every source under ``csrc/`` into objects under
``csrc/_obj/`` (only those older than their sources or any header) and links the shared library
next to this file. nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
OUTPUT = os.path.join(HERE, "libbobcat_cuda.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr"]


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def headers() -> list[str]:
    found = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    found.append(os.path.join(HERE, "..", "include", "bobcat_cuda.h"))
    found.append(os.path.join(HERE, "..", "include", "bobcat_cuda_test.h"))
    return found


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    built = os.path.getmtime(target)
    return any(os.path.getmtime(d) > built for d in deps)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if _stale(obj, [path] + headers()):
        cmd = [NVCC] + ARCH + COMMON + ["-x", "cu", "-c", path, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s\n%s" % (src, result.stdout, result.stderr))
        if verbose or result.stderr.strip():
            sys.stderr.write(result.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for f in os.listdir(OBJ):
            os.remove(os.path.join(OBJ, f))
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(lambda s: _compile(s, verbose), sources()))
    if _stale(OUTPUT, objects):
        cmd = [NVCC] + ARCH + ["-shared", "-o", OUTPUT] + objects + ["-Xlinker", "--exclude-libs,ALL", "-lpthread"]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (result.stdout, result.stderr))
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
