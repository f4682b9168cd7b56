"""Drive the REFERENCE's own CUDA kernels (oracle/_ref, built by build_ref.py) through the
same host mirror as the product library.

TEST INFRASTRUCTURE, NOT PRODUCT. `RefContext` has the `gpu_*` methods `DenseBlock`,
`FeedForwardNetwork` and `Tensor` call, but every one of them launches a kernel of the
reference with the reference's launch configuration (oracle/ref_runner.cu restates
src/io/device/{ffn,util}_device.rs). It is a class of its own: it does not load or call the
product library, so a process that only uses it maps oracle/_ref/libsoklyn_ref.so and nothing
else of this repository. Device memory and the stream come from torch. Used to pin the CPU
oracle against what the reference actually computes, to produce tests/golden/, and as the
benchmark's reference arm.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from soklyn_b200 import log
from soklyn_b200._native import SkDense, SkOptim   # ctypes layouts only; the library is not loaded
from soklyn_b200.core import SK_DTYPE
from soklyn_b200.function import Precision

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_HERE, "_ref", "libsoklyn_ref.so")
PTX = os.path.join(_HERE, "_ref", "nn_math.ptx")


def available() -> bool:
    return os.path.exists(LIB) and os.path.exists(PTX)


def _optim(o) -> SkOptim:
    b1, b2, eps, nest = o.kernel_args()
    return SkOptim(o.ordinal(), b1, b2, eps, nest)


class RefContext:
    """The reference's GpuContext (src/io/device.rs) over its own PTX module.
    sync_each_launch=True reproduces the reference's stream.synchronize() after every launch."""

    def __init__(self, tile_dim: int = 16, ordinal: int = 0, sync_each_launch: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("the reference kernels need a CUDA device")
        if not available():
            raise RuntimeError("reference kernels are not built (python oracle/build_ref.py needs the reference tree)")
        self.device = torch.device("cuda", ordinal)
        self.tile_dim = tile_dim
        torch.cuda.set_device(self.device)
        self.stream = torch.cuda.current_stream(self.device)
        self.ref = C.CDLL(LIB)
        self.ref.ref_load.argtypes = [C.c_char_p]
        self.ref.ref_configure.argtypes = [C.c_void_p, C.c_uint32, C.c_int]
        self.ref.ref_launch_count.restype = C.c_ulonglong
        self.ref.ref_fill.argtypes = [C.c_void_p, C.c_uint32, C.c_float, C.c_size_t]
        self.ref.ref_cast.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_size_t]
        self.ref.ref_dense_forward.argtypes = [C.POINTER(SkDense), C.c_void_p] + [C.c_uint32] * 5
        self.ref.ref_output_error.argtypes = [C.POINTER(SkDense), C.c_void_p] + [C.c_uint32] * 4 + [C.c_float]
        self.ref.ref_hidden_error.argtypes = [C.POINTER(SkDense), C.POINTER(SkDense), C.c_uint32, C.c_uint32]
        self.ref.ref_backward_update.argtypes = [C.POINTER(SkDense), C.c_void_p, C.c_uint32, C.c_uint32,
                                                 C.POINTER(SkOptim), C.POINTER(SkOptim), C.c_float, C.c_float, C.c_uint32]
        if self.ref.ref_load(PTX.encode()) != 0:
            raise RuntimeError("could not load the reference PTX module")
        self.ref.ref_configure(C.c_void_p(self.stream.cuda_stream), tile_dim, int(sync_each_launch))

    # the whole-network calls of the product library do not exist here: every layer goes through
    # the reference kernels below, in the order of src/ffn.rs
    gpu_ffn_forward = None
    gpu_ffn_backward = None

    def close(self):
        self.synchronize()

    def _rc(self, rc):
        if rc != 0:
            raise RuntimeError(f"reference kernel launch failed (status {rc})")

    def synchronize(self):
        self._rc(self.ref.ref_sync())

    def ref_launch_count(self) -> int:
        return int(self.ref.ref_launch_count())

    def get_tile_dim(self) -> int:
        return self.tile_dim

    def download(self, tensor):
        return tensor.download(self)

    def check_tile_dim(self, precision: Precision):
        """src/io/device.rs:248-258"""
        if precision != Precision.FP32 and self.tile_dim != 16:
            raise log.HardwareConstraintViolation(precision, 16, self.tile_dim)

    # -- src/io/device/util_device.rs:7-78 --
    def gpu_cast_t(self, src, dst):
        if src.len() != dst.len():
            raise log.MismatchedDimensions("GPU precision cast source vs destination buffer sizes", dst.len(), src.len())
        rc = self.ref.ref_cast(src.ptr(), SK_DTYPE[src.precision], dst.ptr(), SK_DTYPE[dst.precision], src.len())
        if rc == 8:
            raise log.UnsupportedTypeCast(src.precision, dst.precision)
        self._rc(rc)

    def gpu_broadcast(self, dst, value: float):
        self._rc(self.ref.ref_fill(dst.ptr(), SK_DTYPE[dst.precision], value, dst.len()))

    # -- src/io/device/ffn_device.rs --
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

    def gpu_hidden_layer_backward_pass(self, cur, nxt, input, activation, train_ctx, step):
        """src/io/device/ffn_device.rs:360-439: the delta kernel, then gpu_backward_pass of the same layer."""
        self.gpu_hidden_layer_error(cur, nxt, train_ctx.batch_size)
        self.gpu_backward_pass(cur, input, train_ctx, step)
