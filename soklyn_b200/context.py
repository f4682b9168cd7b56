"""Configuration records of the reference (src/util/context.rs:1-85)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

from .function import Activation, LossFunc, Normalisation, Optimiser, Regularisation

F32_MAX = 3.4028234663852886e38


@dataclass
class LayerInitConfig:
    normalisation: Normalisation = Normalisation.Disabled
    activation: Activation = Activation.Identity
    regularisation: Regularisation = field(default_factory=Regularisation.none)
    mask_coeff: float = 0.0


@dataclass
class TrainContext:
    optimiser: Optimiser
    norm_optimiser: Optimiser
    batch_size: int
    learn_rate: float
    grad_clamp: float = F32_MAX


@dataclass
class MultiLayerTrainContext:
    optimisers: Sequence[Optimiser]
    norm_optimisers: Sequence[Optimiser]
    batch_size: int
    learn_rate: float
    grad_clamp: float = F32_MAX

    def get_train_context(self, idx: int) -> TrainContext:
        return TrainContext(self.optimisers[idx], self.norm_optimisers[idx], self.batch_size,
                            self.learn_rate, self.grad_clamp)


@dataclass
class LossConfig:
    loss_func: LossFunc
    activation: Activation
