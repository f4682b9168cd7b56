"""FeedForwardNetwork of the host mirror (reference: src/ffn.rs)."""
from __future__ import annotations

from typing import List, Sequence

from . import log
from .context import LossConfig, MultiLayerTrainContext
from .core import Tensor
from .function import Precision
from .mlp import DenseBlock


class FeedForwardNetwork:
    def __init__(self, layers: Sequence[DenseBlock], inputs: int):
        self.layers = list(layers)
        self.inputs = inputs

    def forward(self, context, input: Tensor, batch_size: int, use_dropout: bool, step: int,
                row_offset: int = 0) -> List[Tensor]:
        """src/ffn.rs:40-57 — returns every layer's output tensor (borrowed, not copied)."""
        if callable(getattr(context, "gpu_ffn_forward", None)) and self.layers:
            # same checks as DenseBlock::forward, then one native call for the whole stack
            cur = input
            for layer in self.layers:
                layer.check_input_dimension(cur, batch_size)
                layer._check_mode(batch_size)
                cur = layer.get_outputs()
            context.gpu_ffn_forward(self.layers, input, batch_size, use_dropout, step, row_offset)
            return [layer.get_outputs() for layer in self.layers]
        outputs, cur = [], input
        for layer in self.layers:
            cur = layer.forward(context, cur, batch_size, use_dropout, step, row_offset)
            outputs.append(cur)
        return outputs

    def forward_raw(self, context, raw_pixels, batch_size: int, use_dropout: bool, step: int) -> Tensor:
        """src/ffn.rs:73-94 — host vector in, copy of the last layer's output back."""
        if not self.layers:
            raise log.InvalidConfiguration("Cannot execute raw forward pass on an empty network matrix architecture")
        prec = self.layers[0].precision
        x = Tensor.from_cpu_vector(context, raw_pixels, (batch_size, self.inputs), prec)
        return self.forward(context, x, batch_size, use_dropout, step)[-1].clone(context)

    def backward(self, context, outputs: Sequence[Tensor], target: Tensor, input: Tensor, loss_config: LossConfig,
                 train_ctx: MultiLayerTrainContext, step: int):
        """src/ffn.rs:113-166 — output layer first, then the hidden layers in reverse; each
        hidden delta reads the next layer's weights after that layer's update."""
        n = len(self.layers)
        if len(outputs) != n or len(train_ctx.optimisers) != n:
            raise log.InvalidConfiguration(
                f"Backward pass expects exactly {n} activation vectors and optimizers. "
                f"Found {len(outputs)} outputs, {len(train_ctx.optimisers)} optimisers.")
        last = n - 1
        if callable(getattr(context, "gpu_ffn_backward", None)) and all(o is l.get_outputs() for o, l in zip(outputs, self.layers)):
            self._check_backward(target, input, loss_config, train_ctx)
            context.gpu_ffn_backward(self.layers, target, input, loss_config, train_ctx, step)
            return
        head_input = outputs[last - 1] if last > 0 else input
        self.layers[last].compute_loss(context, target, loss_config)
        self.layers[last].backward_output(context, head_input, train_ctx.get_train_context(last), step)
        for i in range(last - 1, -1, -1):
            layer_input = outputs[i - 1] if i > 0 else input
            self.layers[i].backward_hidden(context, self.layers[i + 1], layer_input, train_ctx.get_train_context(i), step)

    def _check_backward(self, target, input, loss_config, train_ctx):
        """The host-side checks of compute_loss / backward_output / backward_hidden (src/mlp.rs:607-821)."""
        from .function import Activation, LossFunc
        last = self.layers[-1]
        if not all(l.is_training_mode() for l in self.layers):
            raise log.TrainingModeRequired("backward pass")
        if target.cols() != last.get_weights().cols():
            raise log.MismatchedDimensions("target columns", last.get_weights().cols(), target.cols())
        if target.rows() > last.get_max_batch_size():
            raise log.AllocationLimitExceeded(target.rows(), last.get_max_batch_size(), "target batches")
        lf, act = loss_config.loss_func, loss_config.activation
        if lf == LossFunc.MeanSquareLoss and act == Activation.Softmax:
            raise log.InvalidConfiguration("Mean Squared Loss does not support the Softmax activation function.")
        if lf == LossFunc.CrossEntropyLoss and act != Activation.Softmax:
            raise log.InvalidConfiguration("Cross-Entropy Loss only supports the Softmax activation function.")
        if lf == LossFunc.BinaryCrossEntropy and act != Activation.Sigmoid:
            raise log.InvalidConfiguration("Binary Cross-Entropy only supports the Sigmoid activation function.")
        cur = input
        for i, layer in enumerate(self.layers):
            layer.check_input_dimension(cur, train_ctx.batch_size)
            layer._check_mode(train_ctx.batch_size)
            if i + 1 < len(self.layers) and self.layers[i + 1].get_weights().rows() != layer.get_weights().cols():
                raise log.MismatchedDimensions("backward pass weight adjacency (next layer rows vs current cols)",
                                               layer.get_weights().cols(), self.layers[i + 1].get_weights().rows())
            cur = layer.get_outputs()

    def get_layers(self):
        return self.layers

    def len(self) -> int:
        return len(self.layers)

    def __len__(self):
        return len(self.layers)

    def is_empty(self) -> bool:
        return not self.layers
