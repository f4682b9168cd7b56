"""Data-parallel training of a FeedForwardNetwork: one process per GPU, batch rows split
across ranks, parameters replicated. No counterpart in the reference (single device).

Forward, loss delta and hidden deltas are independent per row; the only exchange is the sum
over rows of dW, dB and the normalisation-parameter gradients. Because every hidden delta
must read the next layer's weights AFTER that layer's update (src/ffn.rs:141-163), the
order per layer is: local batch sums -> all-reduce (NCCL) -> optimiser step -> delta of the
layer below. Dropout hashes the global row index and every 1/M uses the global batch, so N
ranks reproduce the single-device result up to the order of the f32 sums.

BatchNorm layers would need their column statistics all-reduced as well; that is not built.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from . import log
from .context import LossConfig, MultiLayerTrainContext
from .core import Tensor
from .ffn import FeedForwardNetwork
from .function import Normalisation


def shard_rows(global_batch: int, rank: int, world: int):
    """(first row, row count) of this rank's contiguous shard; the batch must divide evenly."""
    if global_batch % world != 0:
        raise log.InvalidBatchSize(f"global batch {global_batch} is not divisible by {world} ranks")
    per = global_batch // world
    return rank * per, per


class DataParallelFFN:
    def __init__(self, context, network: FeedForwardNetwork, global_batch: int, rank: int, world: int, group=None):
        self.ctx, self.net, self.group = context, network, group
        self.rank, self.world, self.global_batch = rank, world, global_batch
        self.row_offset, self.local_batch = shard_rows(global_batch, rank, world)
        for layer in network.get_layers():
            if layer.get_normalisation() == Normalisation.BatchNorm and world > 1:
                raise log.InvalidConfiguration("BatchNorm is not supported under data parallelism")
        dev = context.device
        layers = network.get_layers() if world > 1 else []
        self.dw = [torch.empty(l.get_weights().rows(), l.get_weights().cols(), device=dev, dtype=torch.float32)
                   for l in layers]
        self.colsums = [torch.empty(3, l.get_weights().cols(), device=dev, dtype=torch.float32) for l in layers]
        self.collectives = 0

    def forward(self, input: Tensor, use_dropout: bool, step: int):
        return self.net.forward(self.ctx, input, self.local_batch, use_dropout, step, self.row_offset)

    def _exchange(self, i: int):
        if self.world > 1:
            dist.all_reduce(self.dw[i], group=self.group)
            dist.all_reduce(self.colsums[i], group=self.group)
            self.collectives += 2

    def backward(self, outputs: Sequence[Tensor], target: Tensor, input: Tensor, loss_config: LossConfig,
                 train_ctx: MultiLayerTrainContext, step: int):
        layers = self.net.get_layers()
        n = len(layers)
        if len(outputs) != n or len(train_ctx.optimisers) != n:
            raise log.InvalidConfiguration(f"Backward pass expects exactly {n} activation vectors and optimizers.")
        if train_ctx.batch_size != self.global_batch:
            raise log.InvalidBatchSize("train context batch size must be the global batch")
        last = n - 1
        layers[last].compute_loss(self.ctx, target, loss_config)
        for i in range(last, -1, -1):
            layer = layers[i]
            x = outputs[i - 1] if i > 0 else input
            if i < last:
                self.ctx.gpu_hidden_layer_error(layer, layers[i + 1], self.local_batch, self.global_batch)
            if self.world == 1:   # nothing to exchange: dW GEMM with the optimiser step in its epilogue
                tc1 = train_ctx.get_train_context(i)
                self.ctx.gpu_backward_pass(layer, x, tc1, step)
                continue
            self.ctx.gpu_backward_grads(layer, x, self.local_batch, self.dw[i], self.colsums[i])
            self._exchange(i)
            self.ctx.gpu_apply_update(layer, self.dw[i], self.colsums[i], self.global_batch,
                                      train_ctx.get_train_context(i), step)
