"""Build the reference's own CUDA kernels and their launcher into oracle/_ref/.

TEST INFRASTRUCTURE, NOT PRODUCT. Needs a checkout of the reference, named by the
environment variable SOKLYN_REF_DIR; nothing is copied from it. Outputs, all git-ignored:
  oracle/_ref/nn_math.ptx        reference src/cuda/nn_math.cu -> compute_75 PTX, the
                                 target of the reference's build.rs:15-18 (`-include
                                 cstdint` supplies uint32_t, which MSVC gets implicitly)
  oracle/_ref/libsoklyn_ref.so   oracle/ref_runner.cu (driver-API launcher)
On a machine without the reference tree the prebuilt files are used as they are.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
PTX = os.path.join(OUT, "nn_math.ptx")
LIB = os.path.join(OUT, "libsoklyn_ref.so")


def _runner_hash() -> str:
    import hashlib
    h = hashlib.sha256()
    for path in (os.path.join(HERE, "ref_runner.cu"), os.path.join(os.path.dirname(HERE), "include", "soklyn_b200.h")):
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def build(force: bool = False, ref_dir: str | None = None) -> bool:
    """PTX from the reference tree (ref_dir, else $SOKLYN_REF_DIR; skipped when neither names one) and
    the launcher library from oracle/ref_runner.cu (rebuilt whenever its sources changed)."""
    ref = ref_dir or os.environ.get("SOKLYN_REF_DIR", "")
    src = os.path.join(ref, "src", "cuda", "nn_math.cu") if ref else ""
    have_ref = bool(src) and os.path.exists(src)
    if not have_ref and not os.path.exists(PTX):
        return False
    os.makedirs(OUT, exist_ok=True)
    if have_ref and (force or not os.path.exists(PTX)):
        subprocess.check_call(["nvcc", "-std=c++17", "-ptx", "-include", "cstdint", "-w",
                               "-gencode", "arch=compute_75,code=compute_75", "-o", PTX, src])
    stamp = LIB + ".hash"
    current = _runner_hash()
    stale = not os.path.exists(LIB) or not os.path.exists(stamp) or open(stamp).read().strip() != current
    if force or stale:
        cuda_home = os.environ.get("CUDA_HOME", os.path.dirname(os.path.dirname(shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")))
        subprocess.check_call(["nvcc", "-std=c++17", "-O2", "-shared", "-Xcompiler", "-fPIC", "-o", LIB,
                               os.path.join(HERE, "ref_runner.cu"), "-L" + os.path.join(cuda_home, "lib64", "stubs"), "-lcuda"])
        with open(stamp, "w") as f:
            f.write(current)
    return os.path.exists(PTX) and os.path.exists(LIB)


if __name__ == "__main__":
    ok = build(force="--force" in sys.argv)
    print("reference kernels:", "built" if ok else "unavailable", OUT)
