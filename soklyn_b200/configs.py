"""The benchmark / parity workloads: network shapes, hyper-parameters and seeded synthetic
data. Shapes follow the reference's examples (Fashion-MNIST 784 features in [0,1],
CIFAR-10 3072 features) but every value is synthetic: numpy PCG64 with fixed seeds,
no dataset item is reproduced.

Seeds: inputs 1000+cfg, labels/targets 2000+cfg, weights 3000+10*cfg+layer.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import List, Optional

import numpy as np

from .context import LayerInitConfig, LossConfig, MultiLayerTrainContext
from .function import Activation, LossFunc, Normalisation, Optimiser, Precision, Regularisation

_ACT = {"identity": Activation.Identity, "sigmoid": Activation.Sigmoid, "relu": Activation.ReLU,
        "tanh": Activation.Tanh, "softmax": Activation.Softmax, "silu": Activation.SiLU, "mish": Activation.Mish}
_NORM = {"disabled": Normalisation.Disabled, "rms": Normalisation.RMSNorm, "layer": Normalisation.LayerNorm,
         "batch": Normalisation.BatchNorm}
_LOSS = {"mse": LossFunc.MeanSquareLoss, "ce": LossFunc.CrossEntropyLoss, "bce": LossFunc.BinaryCrossEntropy}
_PREC = {"f32": Precision.FP32, "f16": Precision.FP16, "bf16": Precision.BF16}


@dataclass(frozen=True)
class NetSpec:
    cfg: int                      # BASELINE config number (seeds derive from it)
    name: str
    dims: tuple                   # layer widths, len = layers + 1
    norms: tuple                  # per layer: disabled / rms / layer / batch
    acts: tuple                   # per layer activation name ("leaky:0.1" for LeakyReLU)
    mask_coeffs: tuple            # per layer dropout probability
    precision: str                # f32 / f16 / bf16
    loss: str                     # mse / ce / bce
    loss_act: str                 # activation applied by compute_loss
    optimiser: str                # "sgd" or "adam"
    lr: float
    batch: int
    init: str                     # he_normal / xavier_normal / xavier_uniform
    inputs: str                   # "u8" (k/255) or "normal"
    targets: str                  # "onehot" / "input" / "normal"
    use_dropout: bool = False
    cosine: Optional[tuple] = None  # (min_lr, max_lr, total, warmup) -> CosineDecayLR

    @property
    def layers(self) -> int:
        return len(self.dims) - 1

    def activation(self, i: int) -> Activation:
        a = self.acts[i]
        return Activation.LeakyReLU(float(a.split(":")[1])) if a.startswith("leaky") else _ACT[a]

    def layer_config(self, i: int) -> LayerInitConfig:
        return LayerInitConfig(_NORM[self.norms[i]], self.activation(i), Regularisation.none(), self.mask_coeffs[i])

    def prec(self) -> Precision:
        return _PREC[self.precision]

    def loss_config(self) -> LossConfig:
        return LossConfig(_LOSS[self.loss], _ACT[self.loss_act])

    def optimisers(self) -> List[Optimiser]:
        o = Optimiser.SGD(0.0, False) if self.optimiser == "sgd" else Optimiser.Adam(0.9, 0.999, 1e-8)
        return [o] * self.layers

    def train_context(self, lr: Optional[float] = None, batch: Optional[int] = None) -> MultiLayerTrainContext:
        return MultiLayerTrainContext(self.optimisers(), self.optimisers(), self.batch if batch is None else batch,
                                      self.lr if lr is None else lr)

    def id_stride(self) -> int:
        """Tensor ids one training block consumes (src/mlp.rs allocation order): 23 in f32, 27 in 16-bit."""
        return 23 if self.precision == "f32" else 27

    def params(self) -> int:
        return sum(self.dims[i] * self.dims[i + 1] for i in range(self.layers))

    def flops_per_step(self, batch: Optional[int] = None) -> float:
        """2MKN for forward and dW of every layer, and for dX of every layer but the first."""
        m = self.batch if batch is None else batch
        f = 0.0
        for i in range(self.layers):
            kn = self.dims[i] * self.dims[i + 1]
            f += 2.0 * m * kn * (2 if i == 0 else 3)
        return f


CONFIGS = {
    1: NetSpec(1, "mlp_784_128_64_10_f32", (784, 128, 64, 10), ("disabled",) * 3, ("relu", "relu", "identity"),
               (0.0,) * 3, "f32", "ce", "softmax", "sgd", 0.01, 64, "he_normal", "u8", "onehot"),
    2: NetSpec(2, "autoencoder_784_256_64_256_784_f16", (784, 256, 64, 256, 784), ("disabled",) * 4,
               ("silu", "silu", "silu", "identity"), (0.0,) * 4, "f16", "mse", "sigmoid", "adam", 1e-3, 256,
               "xavier_normal", "u8", "input"),
    3: NetSpec(3, "classifier_3072_1024_512_10_f16", (3072, 1024, 512, 10), ("layer", "layer", "disabled"),
               ("mish", "mish", "identity"), (0.1, 0.1, 0.0), "f16", "ce", "softmax", "adam", 1e-3, 512,
               "xavier_normal", "normal", "onehot", True, (1e-5, 1e-3, 100, 10)),
    # Adam's learning rate is not named for this configuration; 1e-3 (the autoencoder's) diverges at this width
    # (every step moves each weight by about a tenth of its initial scale: the loss is 0.79, 37.7, ... and NaN
    # by the ninth step), 1e-4 trains (0.79 -> 0.47 in 40 steps).
    4: NetSpec(4, "wide_ffn_4096_16384_x4_f16", (4096, 16384, 4096, 16384, 4096), ("rms", "rms", "rms", "disabled"),
               ("silu", "silu", "silu", "identity"), (0.0,) * 4, "f16", "mse", "identity", "adam", 1e-4, 8192,
               "xavier_uniform", "normal", "normal"),
}


def scaled(spec: NetSpec, dims=None, batch=None, precision=None, name=None) -> NetSpec:
    """Same recipe at other sizes / precision (parity cases that the CPU oracle finishes in seconds)."""
    return replace(spec, dims=tuple(dims) if dims else spec.dims, batch=batch or spec.batch,
                   precision=precision or spec.precision, name=name or spec.name)


def make_weights(spec: NetSpec) -> List[np.ndarray]:
    ws = []
    for i in range(spec.layers):
        k, n = spec.dims[i], spec.dims[i + 1]
        rng = np.random.Generator(np.random.PCG64(3000 + 10 * spec.cfg + i))
        if spec.init == "he_normal":
            w = rng.standard_normal((k, n), dtype=np.float32) * np.float32(math.sqrt(2.0 / k))
        elif spec.init == "xavier_normal":
            w = rng.standard_normal((k, n), dtype=np.float32) * np.float32(math.sqrt(2.0 / (k + n)))
        else:
            lim = np.float32(math.sqrt(6.0 / (k + n)))
            w = (rng.random((k, n), dtype=np.float32) * (2 * lim) - lim).astype(np.float32)
        if spec.precision == "f16":
            w = w.astype(np.float16).astype(np.float32)   # both precisions start from what f16 can hold
        ws.append(np.ascontiguousarray(w))
    return ws


def make_data(spec: NetSpec, batch: Optional[int] = None):
    """(x, target, labels): x [batch x dims[0]], target [batch x dims[-1]] f32; labels or None."""
    m = spec.batch if batch is None else batch
    rx = np.random.Generator(np.random.PCG64(1000 + spec.cfg))
    rt = np.random.Generator(np.random.PCG64(2000 + spec.cfg))
    if spec.inputs == "u8":
        x = rx.integers(0, 256, (m, spec.dims[0])).astype(np.float32) / np.float32(255.0)
    else:
        x = rx.standard_normal((m, spec.dims[0]), dtype=np.float32)
    labels = None
    if spec.targets == "onehot":
        labels = rt.integers(0, spec.dims[-1], m)
        t = np.eye(spec.dims[-1], dtype=np.float32)[labels]
    elif spec.targets == "input":
        t = x.copy()
    else:
        t = rt.standard_normal((m, spec.dims[-1]), dtype=np.float32)
    if spec.precision == "f16":
        x = x.astype(np.float16).astype(np.float32)
        t = t.astype(np.float16).astype(np.float32)
    return np.ascontiguousarray(x), np.ascontiguousarray(t), labels


class _GivenWeights:
    """InitFunc that hands back a prepared matrix (weights are loaded, not drawn)."""

    def __init__(self, w: np.ndarray):
        self.w = w

    def init(self, fan_in, fan_out, length):
        assert self.w.size == length
        return self.w.reshape(-1)


def build_network(context, spec: NetSpec, weights=None, max_batch: Optional[int] = None, is_training: bool = True):
    """FeedForwardNetwork for `spec` on `context`, with explicit weights."""
    from .ffn import FeedForwardNetwork
    from .mlp import DenseBlock
    weights = weights if weights is not None else make_weights(spec)
    mb = spec.batch if max_batch is None else max_batch
    layers = [DenseBlock(context, is_training, spec.dims[i], spec.dims[i + 1], mb, _GivenWeights(weights[i]),
                         spec.layer_config(i), spec.prec()) for i in range(spec.layers)]
    return FeedForwardNetwork(layers, spec.dims[0])


def host_loss(spec: NetSpec, out: np.ndarray, target: np.ndarray) -> float:
    """Scalar loss from the last layer's raw output. The reference never computes one on the
    device (only the delta); this is the same host formula for every implementation."""
    out = out.astype(np.float64)
    t = target.astype(np.float64)
    if spec.loss == "ce":
        z = out - out.max(axis=1, keepdims=True)
        logp = z - np.log(np.exp(z).sum(axis=1, keepdims=True))
        return float(-(t * logp).sum(axis=1).mean())
    if spec.loss_act == "sigmoid":
        out = 1.0 / (1.0 + np.exp(-out))
    if spec.loss == "bce":
        e = 1e-12
        return float(-(t * np.log(out + e) + (1 - t) * np.log(1 - out + e)).mean())
    return float(0.5 * ((out - t) ** 2).mean())
