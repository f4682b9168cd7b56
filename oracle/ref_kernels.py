"""Drive the REFERENCE's own CUDA kernels (oracle/_ref, built by build_ref.py) through the
same host mirror as the product library.

TEST INFRASTRUCTURE, NOT PRODUCT. `RefContext` has the `gpu_*` methods `DenseBlock` and
`FeedForwardNetwork` call, but launches the reference's kernels with the reference's
launch configuration (oracle/ref_runner.cu). Used to pin the CPU oracle against what the
reference actually computes, to produce tests/golden/, and as the benchmark's reference arm.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from soklyn_b200._native import SkDense, SkOptim
from soklyn_b200.device import GpuContext, _optim

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_HERE, "_ref", "libsoklyn_ref.so")
PTX = os.path.join(_HERE, "_ref", "nn_math.ptx")


def available() -> bool:
    return os.path.exists(LIB) and os.path.exists(PTX)


class RefContext(GpuContext):
    """GpuContext whose four hot-path methods run the reference kernels.
    sync_each_launch=True reproduces the reference's stream.synchronize() after every launch."""

    def __init__(self, tile_dim: int = 16, ordinal: int = 0, sync_each_launch: bool = True):
        super().__init__(tile_dim, ordinal)
        if not available():
            raise RuntimeError("reference kernels are not built (python oracle/build_ref.py needs the reference tree)")
        self.ref = C.CDLL(LIB)
        self.ref.ref_load.argtypes = [C.c_char_p]
        self.ref.ref_configure.argtypes = [C.c_void_p, C.c_uint32, C.c_int]
        self.ref.ref_launch_count.restype = C.c_ulonglong
        self.ref.ref_dense_forward.argtypes = [C.POINTER(SkDense), C.c_void_p] + [C.c_uint32] * 5
        self.ref.ref_output_error.argtypes = [C.POINTER(SkDense), C.c_void_p] + [C.c_uint32] * 4 + [C.c_float]
        self.ref.ref_hidden_error.argtypes = [C.POINTER(SkDense), C.POINTER(SkDense), C.c_uint32, C.c_uint32]
        self.ref.ref_backward_update.argtypes = [C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32,
                                                 C.POINTER(SkOptim), C.POINTER(SkOptim), C.c_float, C.c_float, C.c_uint32]
        if self.ref.ref_load(PTX.encode()) != 0:
            raise RuntimeError("could not load the reference PTX module")
        self.ref.ref_configure(C.c_void_p(self.stream.cuda_stream), tile_dim, int(sync_each_launch))

    # the whole-network calls of the product library must not be used: every layer goes through
    # the reference kernels below
    gpu_ffn_forward = None
    gpu_ffn_backward = None

    def _rc(self, rc):
        if rc != 0:
            raise RuntimeError(f"reference kernel launch failed (status {rc})")

    def ref_launch_count(self) -> int:
        return int(self.ref.ref_launch_count())

    def gpu_forward_pass(self, layer, input, batch_size, use_dropout, step, row_offset=0):
        assert row_offset == 0, "the reference is single-device"
        self.check_tile_dim(layer.precision)
        self._rc(self.ref.ref_dense_forward(C.byref(layer.desc()), input.ptr(), input.rows(), batch_size,
                                            int(use_dropout), step & 0xFFFFFFFF, 0))

    def gpu_compute_output_layer_error(self, layer, target, err_mode, activation):
        self._rc(self.ref.ref_output_error(C.byref(layer.desc()), target.ptr(), target.rows(),
                                           layer.get_outputs().rows(), err_mode.value, activation.ordinal(),
                                           activation.coeff))

    def gpu_backward_pass(self, layer, input, train_ctx, step):
        lin, nrm = _optim(train_ctx.optimiser), _optim(train_ctx.norm_optimiser)
        self._rc(self.ref.ref_backward_update(C.byref(layer.desc()), input.ptr(), input.rows(), train_ctx.batch_size,
                                              C.byref(lin), C.byref(nrm), train_ctx.learn_rate, train_ctx.grad_clamp,
                                              step & 0xFFFFFFFF))

    def gpu_hidden_layer_error(self, cur, nxt, batch_size, batch_stat=None):
        self.check_tile_dim(cur.precision)
        self._rc(self.ref.ref_hidden_error(C.byref(cur.desc()), C.byref(nxt.desc()), batch_size, batch_size))
