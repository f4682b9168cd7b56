"""Build the reference's own CUDA kernels and their launcher into oracle/_ref/.

TEST INFRASTRUCTURE, NOT PRODUCT. Needs a checkout of the reference, named by the
environment variable SOKLYN_REF_DIR; nothing is copied from it. Outputs, all git-ignored:
  oracle/_ref/nn_math.ptx        reference src/cuda/nn_math.cu -> compute_75 PTX, the
                                 target of the reference's build.rs:15-18 (`-include
                                 cstdint` supplies uint32_t, which MSVC gets implicitly)
  oracle/_ref/libsoklyn_ref.so   oracle/ref_runner.cu (driver-API launcher)
On a machine without the reference tree the prebuilt files are used as they are.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
PTX = os.path.join(OUT, "nn_math.ptx")
LIB = os.path.join(OUT, "libsoklyn_ref.so")


def build(force: bool = False) -> bool:
    ref = os.environ.get("SOKLYN_REF_DIR", "/root/reference")
    src = os.path.join(ref, "src", "cuda", "nn_math.cu")
    if not os.path.exists(src):
        return os.path.exists(PTX) and os.path.exists(LIB)
    os.makedirs(OUT, exist_ok=True)
    if force or not os.path.exists(PTX):
        subprocess.check_call(["nvcc", "-std=c++17", "-ptx", "-include", "cstdint", "-w",
                               "-gencode", "arch=compute_75,code=compute_75", "-o", PTX, src])
    runner = os.path.join(HERE, "ref_runner.cu")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(runner):
        subprocess.check_call(["nvcc", "-std=c++17", "-O2", "-shared", "-Xcompiler", "-fPIC", "-o", LIB, runner,
                               "-L/usr/local/cuda/lib64/stubs", "-lcuda"])
    return True


if __name__ == "__main__":
    ok = build(force="--force" in sys.argv)
    print("reference kernels:", "built" if ok else "unavailable", OUT)
