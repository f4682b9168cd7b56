"""Build and drive tests/cpp/host_mirror_run.cpp, the test program of the C++ host mirror
(include/soklyn_b200.hpp): write its input file from a NetSpec, parse its output records."""
from __future__ import annotations

import hashlib
import os
import struct
import subprocess

import numpy as np

from soklyn_b200 import _native

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "cpp", "host_mirror_run.cpp")
OUT_DIR = os.path.join(HERE, "cpp", "_build")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")

_NORM = {"disabled": 0, "rms": 1, "layer": 2, "batch": 3}
_ACT = {"identity": 0, "sigmoid": 1, "relu": 2, "leaky": 3, "tanh": 4, "softmax": 5, "silu": 6, "mish": 7}
_LOSS = {"mse": 0, "ce": 1, "bce": 2}
_PREC = {"f32": 0, "f16": 1, "bf16": 2}


def build() -> str:
    """Compile the driver against the in-tree library (rebuilt only when a source changed)."""
    lib = _native.build()
    libdir = os.path.dirname(lib)
    os.makedirs(OUT_DIR, exist_ok=True)
    exe = os.path.join(OUT_DIR, "host_mirror_run")
    h = hashlib.sha256()
    for p in (SRC, os.path.join(ROOT, "include", "soklyn_b200.hpp"), os.path.join(ROOT, "include", "soklyn_b200.h")):
        h.update(open(p, "rb").read())
    stamp = exe + ".hash"
    if os.path.exists(exe) and os.path.exists(stamp) and open(stamp).read() == h.hexdigest():
        return exe
    cmd = ["g++", "-std=c++17", "-O2", "-Wall", "-Wextra", "-Werror", f"-I{ROOT}/include", f"-I{CUDA}/include", SRC, "-o", exe,
           f"-L{libdir}", "-lsoklyn_b200", f"-L{CUDA}/lib64", "-lcudart",
           "-Wl,-rpath,$ORIGIN/../../../soklyn_b200/lib", f"-Wl,-rpath,{CUDA}/lib64"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    open(stamp, "w").write(h.hexdigest())
    return exe


def run(*args, timeout=600) -> subprocess.CompletedProcess:
    return subprocess.run([build(), *args], capture_output=True, text=True, timeout=timeout)


def write_spec(path, spec, weights, x, t, steps, fused=True, max_batch=None):
    u32 = lambda *v: struct.pack(f"<{len(v)}I", *v)
    f32 = lambda *v: struct.pack(f"<{len(v)}f", *v)
    cos = spec.cosine or (0.0, 0.0, 0, 0)
    with open(path, "wb") as f:
        f.write(u32(0x4E4C4B53, _PREC[spec.precision], spec.layers, spec.batch, max_batch or spec.batch, steps,
                    _LOSS[spec.loss], _ACT[spec.loss_act], 0 if spec.optimiser == "sgd" else 1, int(spec.use_dropout),
                    int(fused), int(spec.cosine is not None), cos[2], cos[3]))
        f.write(f32(spec.lr, 0.0, cos[0], cos[1]))
        f.write(u32(*spec.dims))
        for i in range(spec.layers):
            a = spec.acts[i]
            kind, coeff = (3, float(a.split(":")[1])) if a.startswith("leaky") else (_ACT[a], 0.0)
            f.write(u32(_NORM[spec.norms[i]], kind) + f32(coeff, spec.mask_coeffs[i]) + u32(0) + f32(0.0))
        for w in weights:
            f.write(np.ascontiguousarray(w, np.float32).tobytes())
        f.write(np.ascontiguousarray(x[: spec.batch], np.float32).tobytes())
        f.write(np.ascontiguousarray(t[: spec.batch], np.float32).tobytes())


def read_records(path):
    """[(name, f32 array)] in file order."""
    out, buf, pos = [], open(path, "rb").read(), 0
    while pos < len(buf):
        (n,) = struct.unpack_from("<I", buf, pos)
        name = buf[pos + 4: pos + 4 + n].decode()
        (c,) = struct.unpack_from("<Q", buf, pos + 4 + n)
        pos += 12 + n
        out.append((name, np.frombuffer(buf, np.float32, c, pos).copy()))
        pos += 4 * c
    return out
