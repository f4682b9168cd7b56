"""Build and load the CUDA library behind the C ABI (include/soklyn_b200.h).

There is no CPU fallback: importing the library fails loudly when it cannot be built
or loaded, and every compute entry point needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import glob
import hashlib
import os
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG, "csrc")
_LIB = os.path.join(_PKG, "lib", "libsoklyn_b200.so")
_INCLUDE = os.path.join(os.path.dirname(_PKG), "include")

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--split-compile=0",
              "-shared", "-Xcompiler", "-fPIC"]

SK_F32, SK_F16, SK_BF16 = 0, 1, 2

STATUS = {
    0: "ok", 1: "DriverError", 2: "MismatchedDimensions", 3: "AllocationLimitExceeded",
    4: "InvalidConfiguration", 5: "InvalidBatchSize", 6: "TrainingModeRequired",
    7: "HardwareConstraintViolation", 8: "UnsupportedTypeCast", 9: "NullPointer",
    10: "WorkspaceTooSmall", 11: "DeviceTimeout", 12: "StaticScratchLimit",
}


class SkOptim(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("beta1", C.c_float), ("beta2", C.c_float),
                ("epsilon", C.c_float), ("nesterov", C.c_uint32)]


class SkDense(C.Structure):
    _fields_ = (
        [("dtype", C.c_uint32), ("K", C.c_uint32), ("N", C.c_uint32), ("max_batch", C.c_uint32),
         ("is_training", C.c_uint32)]
        + [(n, C.c_void_p) for n in (
            "w", "b", "master_w", "master_b", "dv_w", "dv_b", "dm_w", "dm_b",
            "norm_w", "norm_b", "master_norm_w", "master_norm_b",
            "dv_norm_w", "dv_norm_b", "dm_norm_w", "dm_norm_b",
            "out", "predrop", "preact", "centered", "prenorm", "norm_rstd", "mask",
            "grad", "d_prenorm", "d_norm_w", "d_norm_b", "d_prenorm_lp")]
        + [("norm", C.c_uint32), ("act", C.c_uint32), ("leaky_coeff", C.c_float), ("regu", C.c_uint32),
           ("regu_coeff", C.c_float), ("mask_coeff", C.c_float), ("tensor_id", C.c_uint32)]
    )


class SkExchange(C.Structure):
    """Per-layer pointer tables of sk_dp_backward: arrays of `world` device pointers, one per rank."""
    _fields_ = [("peer_grad", C.c_void_p), ("peer_w", C.c_void_p), ("peer_flags", C.c_void_p), ("peer_colsums", C.c_void_p),
                ("mc_grad", C.c_void_p), ("mc_w", C.c_void_p)]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(_CSRC, "*.cu")))


def _source_hash() -> str:
    h = hashlib.sha256()
    for d in sorted(glob.glob(os.path.join(_CSRC, "*")) + glob.glob(os.path.join(_INCLUDE, "*.h"))):
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _stale() -> bool:
    """True when the built library does not match the sources (by content, so that a
    copy of the tree with new timestamps does not trigger a rebuild)."""
    if not os.path.exists(_LIB) or not os.path.exists(_LIB + ".hash"):
        return True
    with open(_LIB + ".hash") as f:
        return f.read().strip() != _source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/*.cu for sm_100a into soklyn_b200/lib/libsoklyn_b200.so (in-tree)."""
    if force or _stale():
        os.makedirs(os.path.dirname(_LIB), exist_ok=True)
        cmd = ["nvcc", *NVCC_FLAGS, "-o", _LIB, *sources()]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        subprocess.check_call(cmd)
        with open(_LIB + ".hash", "w") as f:
            f.write(_source_hash())
    return _LIB


_lib = None

_SIGS = {
    "sk_ctx_create": (C.c_int, [C.c_int, C.c_uint32, C.c_void_p, C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]),
    "sk_ctx_destroy": (None, [C.c_void_p]),
    "sk_ctx_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "sk_ctx_set_option": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32]),
    "sk_ctx_reserve": (C.c_int, [C.c_void_p, C.c_size_t]),
    "sk_sync": (C.c_int, [C.c_void_p]),
    "sk_status_string": (C.c_char_p, [C.c_int]),
    "sk_last_error": (C.c_char_p, [C.c_void_p]),
    "sk_launch_count": (C.c_uint64, [C.c_void_p]),
    "sk_step_begin": (C.c_int, [C.c_void_p, C.c_uint32]),
    "sk_step_end": (C.c_int, [C.c_void_p]),
    "sk_step_abort": (C.c_int, [C.c_void_p]),
    "sk_step_stats": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "sk_profile_enable": (C.c_int, [C.c_void_p, C.c_int]),
    "sk_profile_read": (C.c_int, [C.c_void_p, C.c_uint32, C.POINTER(C.c_uint64), C.POINTER(C.c_double)]),
    "sk_scramble_seed": (C.c_uint32, [C.c_uint32, C.c_uint32]),
    "sk_dense_forward": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32,
                                   C.c_uint32, C.c_uint32, C.c_uint32]),
    "sk_dense_forward_batchnorm": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32,
                                             C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32]),
    "sk_output_error": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32,
                                  C.c_uint32, C.c_uint32, C.c_float]),
    "sk_hidden_error": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.POINTER(SkDense), C.c_uint32, C.c_uint32]),
    "sk_backward_update": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32,
                                     C.POINTER(SkOptim), C.POINTER(SkOptim), C.c_float, C.c_float, C.c_uint32]),
    "sk_ffn_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                 C.c_uint32, C.c_uint32]),
    "sk_ffn_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32,
                                  C.c_uint32, C.c_uint32, C.c_float, C.c_void_p, C.c_void_p, C.c_uint32, C.c_float,
                                  C.c_float, C.c_uint32]),
    "sk_backward_grads": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32,
                                    C.c_void_p, C.c_void_p]),
    "sk_apply_update": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_void_p, C.c_uint32,
                                  C.POINTER(SkOptim), C.POINTER(SkOptim), C.c_float, C.c_float, C.c_uint32]),
    "sk_backward_grads_lp": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                       C.c_void_p, C.c_void_p]),
    "sk_apply_update_rows": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32,
                                       C.POINTER(SkOptim), C.c_float, C.c_float, C.c_uint32]),
    "sk_apply_vector_update": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.POINTER(SkOptim),
                                         C.POINTER(SkOptim), C.c_float, C.c_float, C.c_uint32]),
    "sk_reduce_update_broadcast": (C.c_int, [C.c_void_p, C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32,
                                             C.c_void_p, C.POINTER(SkOptim), C.c_float, C.c_float, C.c_uint32]),
    "sk_dp_blocks": (C.c_uint32, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "sk_dp_flag_bytes": (C.c_uint32, []),
    "sk_dp_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p,
                                 C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_void_p, C.c_void_p, C.c_uint32,
                                 C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float,
                                 C.c_uint32]),
    "sk_copy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "sk_peer_alloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "sk_peer_open": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "sk_peer_close": (C.c_int, [C.c_void_p, C.c_void_p]),
    "sk_peer_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "sk_signal_peers": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32]),
    "sk_wait_flags": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32]),
    "sk_column_sums_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32,
                                        C.c_uint32, C.c_uint32]),
    "sk_cast": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_size_t]),
    "sk_fill": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_float, C.c_size_t]),
}


def exported_symbols() -> list[str]:
    """Entry points include/soklyn_b200.h declares (kept in step with _SIGS by a test)."""
    return sorted(_SIGS)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        # SOKLYN_B200_LIB points at an alternative build of the same library (kernel experiments)
        path = os.environ.get("SOKLYN_B200_LIB") or (_LIB if os.path.exists(_LIB) and not _stale() else build())
        _lib = C.CDLL(path)
        for name, (res, args) in _SIGS.items():
            fn = getattr(_lib, name)  # AttributeError here = the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
    return _lib
