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
        head_input = outputs[last - 1] if last > 0 else input
        self.layers[last].compute_loss(context, target, loss_config)
        self.layers[last].backward_output(context, head_input, train_ctx.get_train_context(last), step)
        for i in range(last - 1, -1, -1):
            layer_input = outputs[i - 1] if i > 0 else input
            self.layers[i].backward_hidden(context, self.layers[i + 1], layer_input, train_ctx.get_train_context(i), step)

    def get_layers(self):
        return self.layers

    def len(self) -> int:
        return len(self.layers)

    def __len__(self):
        return len(self.layers)

    def is_empty(self) -> bool:
        return not self.layers
