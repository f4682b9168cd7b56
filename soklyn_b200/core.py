"""Device tensors of the host mirror (reference: src/util/core.rs:414-693, src/util/type.rs).

A `Tensor` owns a torch CUDA tensor (PyTorch is the device-memory allocator here), its
shape and a process-wide id. The id of a block's weight tensor seeds the dropout hash
(src/util/core.rs:84-94), so ids are handed out in allocation order like the reference's
global counter.
"""
from __future__ import annotations

import itertools

import numpy as np
import torch

from . import log
from .function import Precision

_ids = itertools.count()

TORCH_DTYPE = {Precision.FP32: torch.float32, Precision.FP16: torch.float16, Precision.BF16: torch.bfloat16}
SK_DTYPE = {Precision.FP32: 0, Precision.FP16: 1, Precision.BF16: 2}
NP_DTYPE = {Precision.FP32: np.float32, Precision.FP16: np.float16}


def reset_tensor_ids(start: int = 0):
    """Restart the id counter (tests use this to reproduce a fresh reference process)."""
    global _ids
    _ids = itertools.count(start)


def scramble_seed(step: int, layer_id: int) -> int:
    """src/util/core.rs:90-94"""
    m = 0xFFFFFFFF
    h = (step * 1103515245 + layer_id) & m
    h = ((h ^ (h >> 16)) * 1103515245) & m
    return h ^ (h >> 15)


class Tensor:
    """Tensor<T, K> with K in {1D, 2D}: row-major device buffer + shape + id."""

    def __init__(self, data: torch.Tensor, precision: Precision, take_id: bool = True):
        assert data.is_cuda and data.is_contiguous()
        self.data = data
        self.precision = precision
        self.id = next(_ids) if take_id else -1

    # -- constructors (core.rs:557-645, 686-692) --
    @staticmethod
    def from_cpu_vector(context, values, shape, precision: Precision = Precision.FP32) -> "Tensor":
        if isinstance(values, torch.Tensor):   # host tensor (pinned for an asynchronous copy)
            if values.numel() != int(np.prod(shape)):
                raise log.MismatchedDimensions("host vector length vs tensor shape", int(np.prod(shape)), values.numel())
            dev = values.reshape(tuple(shape)).to(device=context.device, dtype=TORCH_DTYPE[precision], non_blocking=True)
            return Tensor(dev.contiguous(), precision)
        arr = np.asarray(values)
        if arr.size != int(np.prod(shape)):
            raise log.MismatchedDimensions("host vector length vs tensor shape", int(np.prod(shape)), arr.size)
        host = torch.from_numpy(np.ascontiguousarray(arr.reshape(shape)))
        return Tensor(host.to(device=context.device, dtype=TORCH_DTYPE[precision]).contiguous(), precision)

    @staticmethod
    def zeros(context, shape, precision: Precision = Precision.FP32, take_id: bool = True) -> "Tensor":
        return Tensor(torch.zeros(tuple(shape), device=context.device, dtype=TORCH_DTYPE[precision]), precision, take_id)

    @staticmethod
    def fill(context, shape, value: float, precision: Precision = Precision.FP32) -> "Tensor":
        t = Tensor.zeros(context, shape, precision)
        t.broadcast(context, value)
        return t

    def clone(self, context) -> "Tensor":
        return Tensor(self.data.clone(), self.precision)

    # -- accessors --
    def get_id(self) -> int:
        return self.id

    def rows(self) -> int:
        return self.data.shape[0]

    def cols(self) -> int:
        return self.data.shape[1]

    def len(self) -> int:
        return self.data.numel()

    def ptr(self) -> int:
        return self.data.data_ptr()

    def download(self, context=None) -> np.ndarray:
        """Device -> host copy as a numpy array (bf16 is widened to f32)."""
        if context is not None:
            context.synchronize()
        t = self.data
        if t.dtype == torch.bfloat16:
            t = t.float()
        return t.cpu().numpy()

    # -- device ops routed through the C ABI (core.rs:675-684, type.rs:140-177) --
    def broadcast(self, context, value: float):
        context.gpu_broadcast(self, value)

    def cast(self, context, precision: Precision) -> "Tensor":
        out = Tensor.zeros(context, self.data.shape, precision)
        context.gpu_cast_t(self, out)
        return out


Tensor1D = Tensor
Tensor2D = Tensor
