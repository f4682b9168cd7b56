"""soklyn_b200 — B200 (sm_100a) implementation of Soklyn's DenseBlock / FeedForwardNetwork
hot path behind the reference's own API names. Compute runs only in the CUDA library
(include/soklyn_b200.h); there is no CPU path."""
from .context import LayerInitConfig, LossConfig, MultiLayerTrainContext, TrainContext
from .core import Tensor, Tensor1D, Tensor2D, reset_tensor_ids, scramble_seed
from .device import GpuContext
from .ffn import FeedForwardNetwork
from .function import (Activation, InitHeNormalFunc, InitHeUniformFunc, InitXavierNormalFunc,
                       InitXavierUniformFunc, InitZeroFunc, LossFunc, Normalisation, Optimiser, Precision,
                       Regularisation)
from .mlp import DenseBlock, ParamState
from .scheduler import CosineDecayLR, ExponentialLR, ReduceLROnPlateauScheduler, SchedulerMode
from . import log

__all__ = [n for n in dir() if not n.startswith("_")]
