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
    """InitFunc (function.rs:190-319). The reference draws from rand_chacha's ChaCha8Rng,
    whose source is not part of the reference tree; this mirror draws the same
    distributions from numpy's PCG64 instead, so values differ from a reference run with
    the same seed (load weights explicitly when bit-equal weights are needed)."""

    def __init__(self, seed: int, factor: float = 1.0):
        self.rng = np.random.Generator(np.random.PCG64(seed))
        self.factor = np.float32(factor)

    def _normal(self, total: int, std: float) -> np.ndarray:
        # Box-Muller on two uniform draws, as normal_dist (function.rs:219-234)
        u1 = (self.rng.integers(0, 2**32, total, dtype=np.uint64).astype(np.float32) + np.float32(1.0)) / np.float32(2**32)
        u2 = self.rng.integers(0, 2**32, total, dtype=np.uint64).astype(np.float32) / np.float32(2**32 - 1)
        z = np.sqrt(np.float32(-2.0) * np.log(u1)) * np.cos(np.float32(2.0 * math.pi) * u2)
        return (self.factor * z * np.float32(std)).astype(np.float32)

    def _uniform(self, total: int, limit: float) -> np.ndarray:
        raw = self.rng.integers(0, 2**32, total, dtype=np.uint64).astype(np.float32) / np.float32(2**32 - 1)
        lim = np.float32(limit)
        return (self.factor * (-lim + raw * (np.float32(2.0) * lim))).astype(np.float32)


class InitXavierUniformFunc(_InitBase):
    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return self._uniform(length, math.sqrt(6.0 / (fan_in + fan_out)))


class InitXavierNormalFunc(_InitBase):
    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return self._normal(length, math.sqrt(2.0 / (fan_in + fan_out)))


class InitHeUniformFunc(_InitBase):
    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return self._uniform(length, math.sqrt(6.0 / fan_in))


class InitHeNormalFunc(_InitBase):
    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return self._normal(length, math.sqrt(2.0 / fan_in))


class InitZeroFunc:
    def __init__(self, seed: int = 0, factor: float = 1.0):
        pass

    def init(self, fan_in: int, fan_out: int, length: int) -> np.ndarray:
        return np.zeros(length, np.float32)
