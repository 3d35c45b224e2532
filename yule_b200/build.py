"""In-tree build of the package's native libraries.

* ``libyule_cuda.so``  — the CUDA backend (``csrc/*.cu``), nvcc, sm_100a only.
* ``libyule_synth.so`` — the host-side synthetic tensor generator / quantiser (``csrc/synth.cpp``), g++.

``python -m yule_b200.build`` builds both (``--force`` rebuilds; ``--verbose`` adds ``-Xptxas -v``).
nvcc cross-compiles without a GPU present.
"""

from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
CUDA_SO = os.path.join(HERE, "libyule_cuda.so")
SYNTH_SO = os.path.join(HERE, "libyule_synth.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math=false", "-Xcompiler", "-fPIC", "-Xcompiler", "-O2", "-shared",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the CUDA backend cannot be built")
    return cand


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    """One nvcc process per source file (in parallel), objects under ``csrc/build/``, then one link."""
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    common = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + [
        os.path.join(os.path.dirname(HERE), "include", "yule_cuda.h"), os.path.abspath(__file__)]
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f not in ("--use_fast_math=false", "-shared")]
    jobs = []
    for src in srcs:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src] + common):
            jobs.append([_nvcc()] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj])
    if jobs:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(subprocess.check_call, jobs))
    objs = [os.path.join(objdir, os.path.basename(s)[:-3] + ".o") for s in srcs]
    if force or jobs or _stale(CUDA_SO, objs):
        subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC"] + objs +
                              ["-ldl", "-o", CUDA_SO])
    return CUDA_SO


def build_synth(force: bool = False) -> str:
    src = os.path.join(CSRC, "synth.cpp")
    if force or _stale(SYNTH_SO, [src, os.path.abspath(__file__)]):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-ffp-contract=off",
                               src, "-o", SYNTH_SO])
    return SYNTH_SO


def main(argv: list[str]) -> int:
    force, verbose = "--force" in argv, "--verbose" in argv
    print(build_synth(force))
    print(build_cuda(force, verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
