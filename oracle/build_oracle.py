"""Build recipe for the CPU oracle (test infrastructure, never shipped).

Produces, next to this file:

* ``libyule_oracle.so`` — the C restatement (``yule_oracle.c``, ``yule_oracle_ext.c``, ``yule_oracle_avx2.c``,
  ``yule_oracle_sampler.c``),
  compiled ``-O2 -ffp-contract=off -fno-fast-math`` so f32 sums round like the Rust code.
* ``_ref/libyule_ref_q4k.so`` — Yule's own hand-written AVX2 kernel
  ``yule-core/src/kernels/q4k_gemv_avx2.S`` assembled *unmodified, where it lies* in a checkout of
  the Yule repository, with the flags its ``yule-core/build.rs:18-25`` uses
  (``-mavx2 -mfma -mf16c``).  Only built when such a checkout is reachable: the directory named by
  ``$YULE_REFERENCE_ROOT``, else a ``reference`` directory beside this repository.  No source is
  copied; only the object lands under ``_ref/``.

* ``_ref/qmv_*.cubin`` — Yule's own CUDA matvec kernels ``yule-gpu/kernels/cuda/qmv_{q4_k,q6_k,q4_0,q8_0}.cu``
  compiled *unmodified, where they lie* for sm_100a (the reference compiles the same sources with nvcc at
  start-up, ``yule-gpu/src/cuda/kernels.rs:145-186``).  ``oracle/ref_cuda.py`` launches them with the reference's
  launch shape; they serve as a second pin of the oracle and as the "reference kernel on the same GPU" timing.

Run ``python oracle/build_oracle.py`` (add ``--force`` to rebuild).
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libyule_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libyule_ref_q4k.so")
REF_ASM_RELPATH = os.path.join("yule-core", "src", "kernels", "q4k_gemv_avx2.S")

_CFLAGS = ["-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-Wall", "-Wextra",
           "-std=gnu11", "-pthread"]


def reference_root() -> str | None:
    cand = os.environ.get("YULE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)),
                                                                 "reference")
    return cand if os.path.isfile(os.path.join(cand, REF_ASM_RELPATH)) else None


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force: bool = False) -> str:
    srcs = [os.path.join(HERE, "yule_oracle.c"), os.path.join(HERE, "yule_oracle_ext.c"),
            os.path.join(HERE, "yule_oracle_avx2.c"), os.path.join(HERE, "yule_oracle_sampler.c")]
    deps = srcs + [os.path.join(HERE, "yule_oracle.h"), os.path.abspath(__file__)]
    if force or _stale(ORACLE_SO, deps):
        # The scalar files are built without any -m flag so nothing can be contracted or widened;
        # the AVX2 file needs -mavx2 -mfma for its intrinsics.
        objs = []
        for src, extra in ((srcs[0], []), (srcs[1], []), (srcs[2], ["-mavx2", "-mfma"]), (srcs[3], [])):
            obj = src[:-2] + ".o"
            subprocess.check_call(["gcc", "-c", src, "-o", obj] +
                                  [f for f in _CFLAGS if f != "-shared"] + extra)
            objs.append(obj)
        subprocess.check_call(["gcc", "-shared", "-o", ORACLE_SO] + objs + ["-lm", "-pthread"])
    return ORACLE_SO


def build_ref(force: bool = False) -> str | None:
    """Assemble Yule's q4k_gemv_avx2.S into _ref/ when a Yule checkout is present.

    Returns the path of the shared object (freshly built or already there), or None.
    """
    root = reference_root()
    if root is None:
        return REF_SO if os.path.exists(REF_SO) else None
    src = os.path.join(root, REF_ASM_RELPATH)
    if force or _stale(REF_SO, [src]):
        os.makedirs(REF_DIR, exist_ok=True)
        subprocess.check_call(["gcc", "-shared", "-fPIC", "-mavx2", "-mfma", "-mf16c", "-Wl,-z,noexecstack", src,
                               "-o", REF_SO])
    return REF_SO


REF_CUDA_KERNELS = ("qmv_q4_k", "qmv_q6_k", "qmv_q4_0", "qmv_q8_0")


def build_ref_cuda(force: bool = False) -> list[str]:
    """Compile Yule's qmv_*.cu kernels into _ref/*.cubin (sm_100a) when a Yule checkout and nvcc are present.

    Returns the cubins that exist afterwards (freshly built or left from an earlier build)."""
    import shutil
    root = reference_root()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    out = []
    for name in REF_CUDA_KERNELS:
        cubin = os.path.join(REF_DIR, name + ".cubin")
        if root is not None and os.path.exists(nvcc):
            src = os.path.join(root, "yule-gpu", "kernels", "cuda", name + ".cu")
            if os.path.isfile(src) and (force or _stale(cubin, [src])):
                os.makedirs(REF_DIR, exist_ok=True)
                subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-cubin", src, "-o", cubin])
        if os.path.exists(cubin):
            out.append(cubin)
    return out


def main(argv: list[str]) -> int:
    force = "--force" in argv
    print(build_oracle(force))
    print(build_ref(force) or "(no Yule checkout reachable: _ref not built)")
    print("\n".join(build_ref_cuda(force)) or "(no Yule checkout reachable: reference CUDA kernels not built)")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
