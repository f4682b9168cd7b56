"""DenseBlock of the host mirror (reference: src/mlp.rs).

Same constructor arguments, getters, checks and error behaviour as the reference's
`DenseBlock<T>`; the device work is done by the C ABI through `GpuContext`.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import log
from ._native import SkDense
from .context import LayerInitConfig, LossConfig, TrainContext
from .core import SK_DTYPE, Tensor
from .function import Activation, LossFunc, Normalisation, Precision, Regularisation


class ParamState:
    """w, b and, for training, their f32 masters (16-bit only) and moments (src/mlp.rs:14-110)."""

    def __init__(self, w, b, master_w, master_b, dv_w, dv_b, dm_w, dm_b):
        self.w, self.b, self.master_w, self.master_b = w, b, master_w, master_b
        self.dv_w, self.dv_b, self.dm_w, self.dm_b = dv_w, dv_b, dm_w, dm_b

    @staticmethod
    def new_linear(context, w_vec, w_shape, b_shape, is_training, precision):
        half = precision != Precision.FP32
        delta = lambda shape: Tensor.zeros(context, shape) if is_training else None
        w = Tensor.from_cpu_vector(context, w_vec, w_shape, precision)
        b = Tensor.zeros(context, b_shape, precision)
        # the master copy holds the weights as the 16-bit tensor stores them (mlp.rs:27-43)
        master_w = w.cast(context, Precision.FP32) if half else None
        master_b = Tensor.zeros(context, b_shape) if half else None
        return ParamState(w, b, master_w, master_b, delta(w_shape), delta(b_shape), delta(w_shape), delta(b_shape))

    @staticmethod
    def new_norm(context, shape, is_training, precision):
        half = precision != Precision.FP32
        delta = lambda: Tensor.zeros(context, shape) if is_training else None
        w = Tensor.fill(context, shape, 1.0, precision)
        b = Tensor.zeros(context, shape, precision)
        master_w = Tensor.fill(context, shape, 1.0) if half else None
        master_b = Tensor.zeros(context, shape) if half else None
        return ParamState(w, b, master_w, master_b, delta(), delta(), delta(), delta())

    def cast_f16(self, context, precision=Precision.FP16):
        """ParamState<f32>::cast_f16 (src/mlp.rs:203-220): 16-bit copies of w / b, the f32 values
        become the masters, the moments move over."""
        return ParamState(self.w.clone(context).cast(context, precision), self.b.clone(context).cast(context, precision),
                          self.w.clone(context), self.b.clone(context), self.dv_w, self.dv_b, self.dm_w, self.dm_b)

    def cast_f32(self, context):
        """ParamState<f16>::cast_f32 (src/mlp.rs:185-200): the masters become w / b."""
        return ParamState(self.master_w.clone(context), self.master_b.clone(context), None, None,
                          self.dv_w, self.dv_b, self.dm_w, self.dm_b)

    def validate(self):
        """src/mlp.rs:112-160: shapes of the optional tensors must match w / b."""
        for name, ref in (("master_w", self.w), ("dv_w", self.w), ("dm_w", self.w),
                          ("master_b", self.b), ("dv_b", self.b), ("dm_b", self.b)):
            t = getattr(self, name)
            if t is not None and tuple(t.data.shape) != tuple(ref.data.shape):
                raise log.MismatchedDimensions(f"parameter state tensor {name}", ref.len(), t.len())


class DenseBlock:
    def __init__(self, context, is_training, inputs, outputs, max_batch_size, init, init_config=None,
                 precision: Precision = Precision.FP32):
        """DenseBlock::new / new_with_config (src/mlp.rs:309-375)."""
        if inputs == 0 or outputs == 0:
            raise log.InvalidConfiguration("Input or output size cannot be 0.")
        if max_batch_size == 0:
            raise log.InvalidConfiguration("Batch size cannot be 0.")
        w_vec = init.init(inputs, outputs, inputs * outputs)
        linear = ParamState.new_linear(context, w_vec, (inputs, outputs), (1, outputs), is_training, precision)
        norm = ParamState.new_norm(context, (1, outputs), is_training, precision)
        self._from_tensors(context, is_training, linear, norm, max_batch_size, init_config or LayerInitConfig(), precision)

    @classmethod
    def new_with_config(cls, context, is_training, inputs, outputs, max_batch_size, init, init_config,
                        precision: Precision = Precision.FP32):
        return cls(context, is_training, inputs, outputs, max_batch_size, init, init_config, precision)

    @classmethod
    def from_tensors(cls, context, is_training, linear_state, norm_state, max_batch_size, init_config,
                     precision: Precision = Precision.FP32):
        self = cls.__new__(cls)
        self._from_tensors(context, is_training, linear_state, norm_state, max_batch_size, init_config, precision)
        return self

    def _from_tensors(self, context, is_training, linear_state, norm_state, max_batch_size, cfg, precision):
        """src/mlp.rs:377-427 (allocation order fixes the tensor ids)."""
        linear_state.validate()
        norm_state.validate()
        self.precision = precision
        self.linear_state, self.norm_state = linear_state, norm_state
        wc = linear_state.w.cols()
        shape = (max_batch_size, wc)
        z = lambda: Tensor.zeros(context, shape, precision)
        self.out, self.predrop_out, self.preact_out, self.centered_out, self.prenorm_out = z(), z(), z(), z(), z()
        self.norm_rstd = Tensor.zeros(context, (max(max_batch_size, wc),), precision)
        delta = lambda: Tensor.zeros(context, shape) if is_training else None
        self.grad, self.d_prenorm_out, self.d_norm_w, self.d_norm_b = delta(), delta(), delta(), delta()
        self.mask = Tensor.fill(context, shape, 1.0, precision)
        # 16-bit copy of d_prenorm_out feeding the tensor-core GEMMs; not a reference tensor, takes no id
        self.d_prenorm_lp = (Tensor.zeros(context, shape, precision, take_id=False)
                             if is_training and precision != Precision.FP32 else None)
        self.max_batch_size = max_batch_size
        self.normalisation, self.activation = cfg.normalisation, cfg.activation
        self.regularisation, self.mask_coeff = cfg.regularisation, cfg.mask_coeff
        self.is_training = is_training
        self._desc = None

    # ---- getters / setters (src/mlp.rs:429-480) ----
    def get_weights(self): return self.linear_state.w
    def get_biases(self): return self.linear_state.b
    def get_master_weights(self): return self.linear_state.master_w
    def get_master_biases(self): return self.linear_state.master_b
    def get_dv_weights(self): return self.linear_state.dv_w
    def get_dv_biases(self): return self.linear_state.dv_b
    def get_dm_weights(self): return self.linear_state.dm_w
    def get_dm_biases(self): return self.linear_state.dm_b
    def get_norm_weights(self): return self.norm_state.w
    def get_norm_biases(self): return self.norm_state.b
    def get_master_norm_weights(self): return self.norm_state.master_w
    def get_master_norm_biases(self): return self.norm_state.master_b
    def get_norm_weights_grad(self): return self.d_norm_w
    def get_norm_biases_grad(self): return self.d_norm_b
    def get_dv_norm_weights(self): return self.norm_state.dv_w
    def get_dv_norm_biases(self): return self.norm_state.dv_b
    def get_dm_norm_weights(self): return self.norm_state.dm_w
    def get_dm_norm_biases(self): return self.norm_state.dm_b
    def get_outputs(self): return self.out
    def get_predrop_outputs(self): return self.predrop_out
    def get_preact_outputs(self): return self.preact_out
    def get_centered_outputs(self): return self.centered_out
    def get_prenorm_outputs(self): return self.prenorm_out
    def get_norm_rstd(self): return self.norm_rstd
    def get_grads(self): return self.grad
    def get_delta_prenorm_out(self): return self.d_prenorm_out
    def get_masks(self): return self.mask
    def get_max_batch_size(self): return self.max_batch_size
    def get_mask_coeff(self): return self.mask_coeff
    def get_normalisation(self): return self.normalisation
    def get_activation(self): return self.activation
    def get_regularisation(self): return self.regularisation
    def is_training_mode(self): return self.is_training

    def set_mask_coeff(self, v): self.mask_coeff = v; self._desc = None
    def set_normalisation(self, v): self.normalisation = v; self._desc = None
    def set_activation(self, v): self.activation = v; self._desc = None
    def set_regularisation(self, v): self.regularisation = v; self._desc = None

    def _converted(self, context, linear, norm, precision):
        """Shared body of convert_f16 / convert_f32 (src/mlp.rs:835-888): parameters through the
        ParamState casts, the six forward-cache tensors and the mask through a device cast, the
        f32 gradient tensors move over unchanged. The source block must not be used afterwards."""
        if (precision == Precision.FP32) == (self.precision == Precision.FP32):
            raise log.UnsupportedTypeCast(self.precision, precision)
        blk = DenseBlock.__new__(DenseBlock)
        blk.precision, blk.linear_state, blk.norm_state = precision, linear, norm
        c = lambda t: t.cast(context, precision)
        blk.out, blk.predrop_out, blk.preact_out = c(self.out), c(self.predrop_out), c(self.preact_out)
        blk.centered_out, blk.prenorm_out, blk.norm_rstd = c(self.centered_out), c(self.prenorm_out), c(self.norm_rstd)
        blk.grad, blk.d_prenorm_out, blk.d_norm_w, blk.d_norm_b = self.grad, self.d_prenorm_out, self.d_norm_w, self.d_norm_b
        blk.mask = c(self.mask)
        blk.d_prenorm_lp = (Tensor.zeros(context, tuple(self.out.data.shape), precision, take_id=False)
                            if self.is_training and precision != Precision.FP32 else None)
        blk.max_batch_size = self.max_batch_size
        blk.normalisation, blk.activation = self.normalisation, self.activation
        blk.regularisation, blk.mask_coeff = self.regularisation, self.mask_coeff
        blk.is_training = self.is_training
        blk._desc = None
        return blk

    def convert_f16(self, context, precision: Precision = Precision.FP16) -> "DenseBlock":
        """DenseBlock<f32>::convert_f16 (src/mlp.rs:835-858); `precision` may also name BF16."""
        if self.precision != Precision.FP32:
            raise log.UnsupportedTypeCast(self.precision, precision)
        return self._converted(context, self.linear_state.cast_f16(context, precision),
                               self.norm_state.cast_f16(context, precision), precision)

    def convert_f32(self, context) -> "DenseBlock":
        """DenseBlock<f16>::convert_f32 (src/mlp.rs:861-888)."""
        if self.precision == Precision.FP32:
            raise log.UnsupportedTypeCast(self.precision, Precision.FP32)
        return self._converted(context, self.linear_state.cast_f32(context), self.norm_state.cast_f32(context),
                               Precision.FP32)

    def reset_mask(self, context):
        self.mask.broadcast(context, 1.0)

    def desc(self) -> SkDense:
        """The block as the C ABI sees it: borrowed device pointers + configuration."""
        if self._desc is None:
            p = lambda t: t.ptr() if t is not None else None
            ls, ns = self.linear_state, self.norm_state
            d = SkDense()
            d.dtype, d.K, d.N = SK_DTYPE[self.precision], ls.w.rows(), ls.w.cols()
            d.max_batch, d.is_training = self.max_batch_size, int(self.is_training)
            d.w, d.b, d.master_w, d.master_b = p(ls.w), p(ls.b), p(ls.master_w), p(ls.master_b)
            d.dv_w, d.dv_b, d.dm_w, d.dm_b = p(ls.dv_w), p(ls.dv_b), p(ls.dm_w), p(ls.dm_b)
            d.norm_w, d.norm_b, d.master_norm_w, d.master_norm_b = p(ns.w), p(ns.b), p(ns.master_w), p(ns.master_b)
            d.dv_norm_w, d.dv_norm_b, d.dm_norm_w, d.dm_norm_b = p(ns.dv_w), p(ns.dv_b), p(ns.dm_w), p(ns.dm_b)
            d.out, d.predrop, d.preact = p(self.out), p(self.predrop_out), p(self.preact_out)
            d.centered, d.prenorm, d.norm_rstd, d.mask = p(self.centered_out), p(self.prenorm_out), p(self.norm_rstd), p(self.mask)
            d.grad, d.d_prenorm, d.d_norm_w, d.d_norm_b = p(self.grad), p(self.d_prenorm_out), p(self.d_norm_w), p(self.d_norm_b)
            d.d_prenorm_lp = p(self.d_prenorm_lp)
            d.norm, d.act, d.leaky_coeff = self.normalisation.ordinal(), self.activation.ordinal(), self.activation.coeff
            d.regu, d.regu_coeff = self.regularisation.ordinal(), self.regularisation.regu_coeff
            d.mask_coeff, d.tensor_id = self.mask_coeff, ls.w.get_id() & 0xFFFFFFFF
            self._desc = d
        return self._desc

    # ---- checks (src/mlp.rs:492-519) ----
    def check_input_dimension(self, input: Tensor, batch_size: int):
        if input.rows() < batch_size:
            raise log.MismatchedDimensions("forward input rows vs explicit batch size", batch_size, input.rows())
        if input.rows() > self.max_batch_size:
            raise log.AllocationLimitExceeded(input.rows(), self.max_batch_size, "input batches")
        if input.cols() != self.linear_state.w.rows():
            raise log.MismatchedDimensions("forward input feature columns mismatch", self.linear_state.w.rows(), input.cols())

    def _check_mode(self, batch_size: int):
        if self.activation == Activation.Softmax:
            raise log.InvalidConfiguration("Softmax activation can only be passed into the compute_loss function.")
        if batch_size == 0:
            raise log.InvalidBatchSize("Batch size must be more than zero.")
        if self.normalisation == Normalisation.BatchNorm and batch_size == 1:
            raise log.InvalidBatchSize("Normalisation is set to BatchNorm, but given batch size is 1. "
                                       "Batch size must be more than 1.")

    # ---- hot path (src/mlp.rs:548-821) ----
    def forward(self, context, input: Tensor, batch_size: int, use_dropout: bool, step: int, row_offset: int = 0) -> Tensor:
        self.check_input_dimension(input, batch_size)
        self._check_mode(batch_size)
        context.gpu_forward_pass(self, input, batch_size, use_dropout, step, row_offset)
        return self.out

    def backward_output(self, context, input: Tensor, train_ctx: TrainContext, step: int):
        if not self.is_training:
            raise log.TrainingModeRequired("output layer backward pass")
        self.check_input_dimension(input, train_ctx.batch_size)
        self._check_mode(train_ctx.batch_size)
        context.gpu_backward_pass(self, input, train_ctx, step)

    def backward_hidden(self, context, next_layer: "DenseBlock", input: Tensor, train_ctx: TrainContext, step: int):
        if not self.is_training:
            raise log.TrainingModeRequired("hidden layer backward pass")
        self.check_input_dimension(input, train_ctx.batch_size)
        cur_cols, next_rows = self.linear_state.w.cols(), next_layer.get_weights().rows()
        if next_rows != cur_cols:
            raise log.MismatchedDimensions("backward pass weight adjacency (next layer rows vs current cols)", cur_cols, next_rows)
        if next_layer.get_grads().rows() < input.rows():
            raise log.MismatchedDimensions("backward pass activation gradient rows should be more than or equal to batch rows",
                                           input.rows(), next_layer.get_grads().rows())
        self._check_mode(train_ctx.batch_size)
        context.gpu_hidden_layer_backward_pass(self, next_layer, input, self.activation, train_ctx, step)

    def compute_loss(self, context, target: Tensor, loss_config: LossConfig):
        if not self.is_training:
            raise log.TrainingModeRequired("compute loss")
        if target.cols() != self.linear_state.w.cols():
            raise log.MismatchedDimensions("target columns", self.linear_state.w.cols(), target.cols())
        if target.rows() > self.max_batch_size:
            raise log.AllocationLimitExceeded(target.rows(), self.max_batch_size, "target batches")
        lf, act = loss_config.loss_func, loss_config.activation
        if lf == LossFunc.MeanSquareLoss and act == Activation.Softmax:
            raise log.InvalidConfiguration("Mean Squared Loss does not support the Softmax activation function.")
        if lf == LossFunc.CrossEntropyLoss and act != Activation.Softmax:
            raise log.InvalidConfiguration("Cross-Entropy Loss only supports the Softmax activation function.")
        if lf == LossFunc.BinaryCrossEntropy and act != Activation.Sigmoid:
            raise log.InvalidConfiguration("Binary Cross-Entropy only supports the Sigmoid activation function.")
        context.gpu_compute_output_layer_error(self, target, lf, act)
