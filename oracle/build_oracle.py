"""Build recipe for the CPU oracle (test infrastructure, never shipped).

Produces, next to this file:

* ``libyule_oracle.so`` — the C restatement (``yule_oracle.c`` + ``yule_oracle_avx2.c``),
  compiled ``-O2 -ffp-contract=off -fno-fast-math`` so f32 sums round like the Rust code.
* ``_ref/libyule_ref_q4k.so`` — Yule's own hand-written AVX2 kernel
  ``yule-core/src/kernels/q4k_gemv_avx2.S`` assembled *unmodified, where it lies* in a checkout of
  the Yule repository, with the flags its ``yule-core/build.rs:18-25`` uses
  (``-mavx2 -mfma -mf16c``).  Only built when such a checkout is reachable: the directory named by
  ``$YULE_REFERENCE_ROOT``, else a ``reference`` directory beside this repository.  No source is
  copied; only the object lands under ``_ref/``.

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
            os.path.join(HERE, "yule_oracle_avx2.c")]
    deps = srcs + [os.path.join(HERE, "yule_oracle.h"), os.path.abspath(__file__)]
    if force or _stale(ORACLE_SO, deps):
        # The scalar files are built without any -m flag so nothing can be contracted or widened;
        # the AVX2 file needs -mavx2 -mfma for its intrinsics.
        objs = []
        for src, extra in ((srcs[0], []), (srcs[1], []), (srcs[2], ["-mavx2", "-mfma"])):
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


def main(argv: list[str]) -> int:
    force = "--force" in argv
    print(build_oracle(force))
    print(build_ref(force) or "(no Yule checkout reachable: _ref not built)")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
