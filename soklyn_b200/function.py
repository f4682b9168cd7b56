"""Hyper-parameter types of the reference (src/util/function.rs:1-319): enums whose
ordinals are the kernel ABI, and the weight initialisers."""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum

import numpy as np


class Precision(Enum):
    FP32 = 0
    FP16 = 1
    BF16 = 2   # extension of this build; the reference has FP32 and FP16


@dataclass(frozen=True)
class Regularisation:
    """None_ / L1Regular{regu_coeff} / L2Regular{regu_coeff} (function.rs:8-41)."""
    kind: int = 0
    regu_coeff: float = 0.0

    @staticmethod
    def none():
        return Regularisation(0, 0.0)

    @staticmethod
    def l1(regu_coeff: float):
        return Regularisation(1, regu_coeff)

    @staticmethod
    def l2(regu_coeff: float):
        return Regularisation(2, regu_coeff)

    def ordinal(self) -> int:
        return self.kind


class Normalisation(Enum):
    """function.rs:45-73"""
    Disabled = 0
    RMSNorm = 1
    LayerNorm = 2
    BatchNorm = 3

    def ordinal(self) -> int:
        return self.value


@dataclass(frozen=True)
class Optimiser:
    """SGD{v_coeff, nesterov} (ordinal 0) / Adam{m_coeff, v_coeff, epsilon} (ordinal 1), function.rs:76-116."""
    kind: int
    m_coeff: float = 0.0
    v_coeff: float = 0.0
    epsilon: float = 0.0
    nesterov: bool = False

    @staticmethod
    def SGD(v_coeff: float = 0.0, nesterov: bool = False):
        return Optimiser(0, 0.0, v_coeff, 0.0, nesterov)

    @staticmethod
    def Adam(m_coeff: float = 0.9, v_coeff: float = 0.999, epsilon: float = 1e-8):
        return Optimiser(1, m_coeff, v_coeff, epsilon, False)

    def ordinal(self) -> int:
        return self.kind

    def kernel_args(self):
        """(beta1, beta2, epsilon, nesterov) as src/io/device/ffn_device.rs:254-264 unpacks them."""
        if self.kind == 0:
            return (self.v_coeff, 0.0, 0.0, int(self.nesterov))
        return (self.m_coeff, self.v_coeff, self.epsilon, 0)


@dataclass(frozen=True)
class Activation:
    """function.rs:119-165; LeakyReLU carries its coefficient."""
    kind: int
    coeff: float = 0.0

    def ordinal(self) -> int:
        return self.kind

    @staticmethod
    def LeakyReLU(coeff: float):
        return Activation(3, coeff)


Activation.Identity = Activation(0)
Activation.Sigmoid = Activation(1)
Activation.ReLU = Activation(2)
Activation.Tanh = Activation(4)
Activation.Softmax = Activation(5)
Activation.SiLU = Activation(6)
Activation.Mish = Activation(7)


class LossFunc(Enum):
    """function.rs:168-176 (`as u32`)."""
    MeanSquareLoss = 0
    CrossEntropyLoss = 1
    BinaryCrossEntropy = 2


class _InitBase:
    """InitFunc (function.rs:190-319): ChaCha8Rng::seed_from_u64(seed), then normal_dist / uniform_dist
    (function.rs:219-248) in f32 arithmetic, operation for operation. The generator is restated in
    soklyn_b200/chacha.py from the published algorithms (the crates' sources are not part of the reference
    tree): its block function is pinned by a known-answer vector, the seed expansion and the f32
    transcendental functions (which follow the platform's libm in the reference) are not, so values can
    differ from a reference run in the last bit. Load weights explicitly when bit-equal weights are needed."""

    _TWO32 = np.float32(4294967296.0)   # `u32::MAX as f32`, and `u32::MAX as f32 + 1.0`, after rounding

    def __init__(self, seed: int, factor: float = 1.0):
        from .chacha import ChaCha8Rng
        self.rng = ChaCha8Rng.seed_from_u64(seed)
        self.factor = np.float32(factor)

    def _normal(self, total: int, std: float) -> np.ndarray:
        draws = self.rng.next_u32s(2 * total)        # element i takes draws 2i (u1) and 2i + 1 (u2)
        u1 = (draws[0::2].astype(np.float32) + np.float32(1.0)) / self._TWO32
        u2 = draws[1::2].astype(np.float32) / self._TWO32
        z = np.sqrt(np.float32(-2.0) * np.log(u1)) * np.cos((np.float32(2.0) * np.float32(math.pi)) * u2)
        return ((self.factor * z) * np.float32(std)).astype(np.float32)

    def _uniform(self, total: int, limit: float) -> np.ndarray:
        raw = self.rng.next_u32s(total).astype(np.float32) / self._TWO32
        lim = np.float32(limit)
        return (self.factor * (-lim + raw * (np.float32(2.0) * lim))).astype(np.float32)


class InitXavierUniformFunc(_InitBase):
    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return self._uniform(length, np.sqrt(np.float32(6.0) / np.float32(fan_in + fan_out)))


class InitXavierNormalFunc(_InitBase):
    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return self._normal(length, np.sqrt(np.float32(2.0) / np.float32(fan_in + fan_out)))


class InitHeUniformFunc(_InitBase):
    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return self._uniform(length, np.sqrt(np.float32(6.0) / np.float32(fan_in)))


class InitHeNormalFunc(_InitBase):
    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return self._normal(length, np.sqrt(np.float32(2.0) / np.float32(fan_in)))


class InitZeroFunc:
    def __init__(self, seed: int = 0, factor: float = 1.0):
        pass

    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return np.zeros(length, np.float32)
