"""GpuContext of the host mirror (reference: src/io/device.rs and src/io/device/{ffn,util}_device.rs).

Each `gpu_*` method is one call into the C ABI (include/soklyn_b200.h), in place of the
reference's kernel-by-name launches. Calls are ordered on this context's stream, which is
torch's current stream at construction unless one is given; unlike the reference the
methods do not block the host, `synchronize()` does.
"""
from __future__ import annotations

import contextlib
import ctypes as C

import torch

from . import _native, log
from ._native import SkDense, SkOptim
from .core import SK_DTYPE, Tensor
from .function import Activation, LossFunc, Normalisation, Optimiser, Precision


def _optim(o: Optimiser) -> SkOptim:
    b1, b2, eps, nest = o.kernel_args()
    return SkOptim(o.ordinal(), b1, b2, eps, nest)


class GpuContext:
    def __init__(self, tile_dim: int = 16, ordinal: int = 0, stream: "torch.cuda.Stream | None" = None,
                 workspace_bytes: int = 0):
        if not torch.cuda.is_available():
            raise log.DriverError("Failed to create CUDA context: no CUDA device (there is no CPU path)")
        self.lib = _native.lib()
        self.device = torch.device("cuda", ordinal)
        self.tile_dim = tile_dim
        torch.cuda.set_device(self.device)
        self.stream = stream if stream is not None else torch.cuda.current_stream(self.device)
        handle = C.c_void_p()
        rc = self.lib.sk_ctx_create(ordinal, tile_dim, C.c_void_p(self.stream.cuda_stream), 0, workspace_bytes,
                                    C.byref(handle))
        if rc != 0:
            raise log.DriverError(f"sk_ctx_create failed with status {rc} ({_native.STATUS.get(rc)})")
        self.handle = handle

    @staticmethod
    def new(tile_dim: int) -> "GpuContext":
        return GpuContext(tile_dim, 0)

    @staticmethod
    def with_device_index(ordinal: int, tile_dim: int) -> "GpuContext":
        return GpuContext(tile_dim, ordinal)

    def close(self):
        if getattr(self, "handle", None):
            self.lib.sk_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- helpers --
    def _check(self, rc: int):
        if rc != 0:
            log.raise_status(rc, self.lib.sk_last_error(self.handle).decode())

    def set_stream(self, stream: "torch.cuda.Stream"):
        self.stream = stream
        self._check(self.lib.sk_ctx_set_stream(self.handle, C.c_void_p(stream.cuda_stream)))

    def set_gemm_engine(self, ffma_only: bool):
        """Force the FFMA GEMM (True) or let the library pick the tensor-core kernel where it can (False)."""
        self._check(self.lib.sk_ctx_set_option(self.handle, 0, int(ffma_only)))

    def set_colsum_handover(self, on: bool):
        """Let gpu_hidden_layer_error hand the layer's column sums to the weight-gradient call that
        follows it directly (the caller must not touch d_prenorm / d_norm_w / d_norm_b in between)."""
        self._check(self.lib.sk_ctx_set_option(self.handle, 1, int(on)))

    def set_lean_backward(self, on: bool):
        """Hidden blocks whose column sums are taken in the dX epilogue stop storing grad, the f32 d_prenorm,
        d_norm_w and d_norm_b (a documented deviation from the reference's API-visible tensors)."""
        self._check(self.lib.sk_ctx_set_option(self.handle, 2, int(on)))

    def set_f32_tensor_cores(self, on: bool):
        """Large f32 products on the tensor cores (three bf16 parts per operand, six partial products, summed
        over K in registers); needs 6 bytes of workspace per operand element (`reserve`)."""
        self._check(self.lib.sk_ctx_set_option(self.handle, 4, int(on)))

    def set_reserve_sms(self, count: int):
        """SMs the tensor-core GEMMs leave free for a kernel on another stream."""
        self._check(self.lib.sk_ctx_set_option(self.handle, 3, int(count)))

    def reserve(self, workspace_bytes: int):
        self._check(self.lib.sk_ctx_reserve(self.handle, workspace_bytes))

    def synchronize(self):
        self._check(self.lib.sk_sync(self.handle))

    def launch_count(self) -> int:
        return int(self.lib.sk_launch_count(self.handle))

    @contextlib.contextmanager
    def step_graph(self, slot: int = 0):
        """Record the calls made inside the block (one training step: forward, backward) and launch them as one
        CUDA graph when the block ends; results are those of the same calls made outside. For the small,
        launch-bound networks. Inside the block nothing may wait for the stream or read a tensor back; the first
        step of a slot runs unrecorded. `slot` names the executable graph that is reused from step to step."""
        self._check(self.lib.sk_step_begin(self.handle, slot))
        try:
            yield
        except BaseException:
            self.lib.sk_step_abort(self.handle)
            raise
        self._check(self.lib.sk_step_end(self.handle))

    def step_graph_stats(self) -> dict:
        out = (C.c_uint64 * 4)()
        self._check(self.lib.sk_step_stats(self.handle, out))
        return dict(zip(("instantiated", "updated", "launched", "unrecorded"), (int(v) for v in out)))

    PROFILE_CLASSES = ("gemm_forward", "gemm_dx", "gemm_dw", "norm", "output_error", "colsum", "update", "exchange")

    def profile_enable(self, on: bool = True):
        self._check(self.lib.sk_profile_enable(self.handle, int(on)))

    def profile_read(self) -> dict:
        """{class: (launches, total_ms)} since profile_enable(True); waits for the stream."""
        out = {}
        for i, name in enumerate(self.PROFILE_CLASSES):
            n, ms = C.c_uint64(), C.c_double()
            self._check(self.lib.sk_profile_read(self.handle, i, C.byref(n), C.byref(ms)))
            out[name] = (n.value, ms.value)
        return out

    def get_tile_dim(self) -> int:
        return self.tile_dim

    def download(self, tensor: Tensor):
        return tensor.download(self)

    def check_tile_dim(self, precision: Precision):
        """src/io/device.rs:248-258"""
        if precision != Precision.FP32 and self.tile_dim != 16:
            raise log.HardwareConstraintViolation(precision, 16, self.tile_dim)

    # -- src/io/device/util_device.rs:7-78 --
    def gpu_cast_t(self, src: Tensor, dst: Tensor):
        if src.len() != dst.len():
            raise log.MismatchedDimensions("GPU precision cast source vs destination buffer sizes", dst.len(), src.len())
        if (src.precision == Precision.FP32) == (dst.precision == Precision.FP32):
            raise log.UnsupportedTypeCast(src.precision, dst.precision)
        self._check(self.lib.sk_cast(self.handle, src.ptr(), SK_DTYPE[src.precision], dst.ptr(),
                                     SK_DTYPE[dst.precision], src.len()))

    def gpu_broadcast(self, dst: Tensor, value: float):
        self._check(self.lib.sk_fill(self.handle, dst.ptr(), SK_DTYPE[dst.precision], value, dst.len()))

    # -- src/io/device/ffn_device.rs --
    def gpu_forward_pass(self, layer, input: Tensor, batch_size: int, use_dropout: bool, step: int,
                         row_offset: int = 0):
        self.check_tile_dim(layer.precision)
        self._check(self.lib.sk_dense_forward(self.handle, C.byref(layer.desc()), input.ptr(), input.rows(),
                                              batch_size, int(use_dropout), step & 0xFFFFFFFF, row_offset))

    def gpu_forward_batchnorm_phase(self, layer, input: Tensor, batch_size: int, batch_stat: int, phase: int,
                                    stats: torch.Tensor, use_dropout: bool, step: int, row_offset: int = 0):
        """One of the three phases of a BatchNorm forward whose batch is split over ranks; `stats` is an
        f32 [2 x N] device tensor the caller sums over ranks between the phases."""
        self.check_tile_dim(layer.precision)
        self._check(self.lib.sk_dense_forward_batchnorm(self.handle, C.byref(layer.desc()), input.ptr(), input.rows(),
                                                        batch_size, batch_stat, phase, stats.data_ptr(),
                                                        int(use_dropout), step & 0xFFFFFFFF, row_offset))

    def gpu_compute_output_layer_error(self, layer, target: Tensor, err_mode: LossFunc, activation: Activation):
        rows = layer.get_outputs().rows()
        self._check(self.lib.sk_output_error(self.handle, C.byref(layer.desc()), target.ptr(), target.rows(), rows,
                                             err_mode.value, activation.ordinal(), activation.coeff))

    def gpu_backward_pass(self, layer, input: Tensor, train_ctx, step: int):
        lin, nrm = _optim(train_ctx.optimiser), _optim(train_ctx.norm_optimiser)
        self._check(self.lib.sk_backward_update(self.handle, C.byref(layer.desc()), input.ptr(), input.rows(),
                                                train_ctx.batch_size, C.byref(lin), C.byref(nrm),
                                                train_ctx.learn_rate, train_ctx.grad_clamp, step & 0xFFFFFFFF))

    def gpu_hidden_layer_error(self, cur, nxt, batch_size: int, batch_stat: int | None = None):
        self.check_tile_dim(cur.precision)
        self._check(self.lib.sk_hidden_error(self.handle, C.byref(cur.desc()), C.byref(nxt.desc()), batch_size,
                                             batch_size if batch_stat is None else batch_stat))

    def gpu_hidden_layer_backward_pass(self, cur, nxt, input: Tensor, activation, train_ctx, step: int):
        self.gpu_hidden_layer_error(cur, nxt, train_ctx.batch_size)
        self.gpu_backward_pass(cur, input, train_ctx, step)

    # -- data-parallel halves (no counterpart in the reference) --
    def gpu_backward_grads(self, layer, input: Tensor, batch_size: int, dw: torch.Tensor, colsums: torch.Tensor):
        self._check(self.lib.sk_backward_grads(self.handle, C.byref(layer.desc()), input.ptr(), input.rows(),
                                               batch_size, dw.data_ptr(), colsums.data_ptr()))

    def gpu_apply_update(self, layer, dw: torch.Tensor, colsums: torch.Tensor, batch_stat: int, train_ctx, step: int):
        lin, nrm = _optim(train_ctx.optimiser), _optim(train_ctx.norm_optimiser)
        self._check(self.lib.sk_apply_update(self.handle, C.byref(layer.desc()), dw.data_ptr(), colsums.data_ptr(),
                                             batch_stat, C.byref(lin), C.byref(nrm), train_ctx.learn_rate,
                                             train_ctx.grad_clamp, step & 0xFFFFFFFF))

    def gpu_backward_grads_lp(self, layer, input: Tensor, batch_size: int, batch_stat: int, grad, colsums: torch.Tensor):
        """grad: a torch tensor or a raw device pointer of T [K x N]."""
        gptr = grad if isinstance(grad, int) else grad.data_ptr()
        self._check(self.lib.sk_backward_grads_lp(self.handle, C.byref(layer.desc()), input.ptr(), input.rows(),
                                                  batch_size, batch_stat, C.c_void_p(gptr), colsums.data_ptr()))

    def gpu_apply_update_rows(self, layer, grad: torch.Tensor, row0: int, nrows: int, train_ctx, step: int):
        lin = _optim(train_ctx.optimiser)
        self._check(self.lib.sk_apply_update_rows(self.handle, C.byref(layer.desc()), grad.data_ptr(), row0, nrows,
                                                  C.byref(lin), train_ctx.learn_rate, train_ctx.grad_clamp,
                                                  step & 0xFFFFFFFF))

    def gpu_apply_vector_update(self, layer, colsums: torch.Tensor, batch_stat: int, train_ctx, step: int):
        lin, nrm = _optim(train_ctx.optimiser), _optim(train_ctx.norm_optimiser)
        self._check(self.lib.sk_apply_vector_update(self.handle, C.byref(layer.desc()), colsums.data_ptr(), batch_stat,
                                                    C.byref(lin), C.byref(nrm), train_ctx.learn_rate,
                                                    train_ctx.grad_clamp, step & 0xFFFFFFFF))

    # -- whole-network calls (src/ffn.rs sequencing done natively) --
    def gpu_ffn_forward(self, layers, input: Tensor, batch_size: int, use_dropout: bool, step: int, row_offset: int = 0):
        self.check_tile_dim(layers[0].precision)
        ptrs = (C.c_void_p * len(layers))(*[C.addressof(l.desc()) for l in layers])
        self._check(self.lib.sk_ffn_forward(self.handle, ptrs, len(layers), input.ptr(), input.rows(), batch_size,
                                            int(use_dropout), step & 0xFFFFFFFF, row_offset))

    def gpu_ffn_backward(self, layers, target: Tensor, input: Tensor, loss_config, train_ctx, step: int):
        n = len(layers)
        ptrs = (C.c_void_p * n)(*[C.addressof(l.desc()) for l in layers])
        lin = (SkOptim * n)(*[_optim(o) for o in train_ctx.optimisers])
        nrm = (SkOptim * n)(*[_optim(o) for o in train_ctx.norm_optimisers])
        act = loss_config.activation
        self._check(self.lib.sk_ffn_backward(self.handle, ptrs, n, target.ptr(), target.rows(), input.ptr(), input.rows(),
                                             loss_config.loss_func.value, act.ordinal(), act.coeff, lin, nrm,
                                             train_ctx.batch_size, train_ctx.learn_rate, train_ctx.grad_clamp,
                                             step & 0xFFFFFFFF))

    # -- data-parallel backward: the whole pass in one native call --
    def dp_blocks(self, k: int, n: int, world: int, wanted: int) -> int:
        return int(self.lib.sk_dp_blocks(k, n, world, wanted))

    def dp_flag_bytes(self) -> int:
        return int(self.lib.sk_dp_flag_bytes())

    def gpu_dp_backward(self, layers, tables, target: Tensor, input: Tensor, loss_config, train_ctx, batch: int,
                        batch_stat: int, world: int, rank: int, blocks: int, epoch: int, step: int):
        n = len(layers)
        ptrs = (C.c_void_p * n)(*[C.addressof(l.desc()) for l in layers])
        lin = (SkOptim * n)(*[_optim(o) for o in train_ctx.optimisers])
        nrm = (SkOptim * n)(*[_optim(o) for o in train_ctx.norm_optimisers])
        act = loss_config.activation
        self._check(self.lib.sk_dp_backward(self.handle, ptrs, tables, n, target.ptr(), target.rows(), input.ptr(),
                                            input.rows(), loss_config.loss_func.value, act.ordinal(), act.coeff, lin, nrm,
                                            batch, batch_stat, world, rank, blocks, epoch & 0xFFFFFFFF,
                                            train_ctx.learn_rate, train_ctx.grad_clamp, step & 0xFFFFFFFF))

    # -- fused exchange over peer-mapped buffers (no counterpart in the reference) --
    def gpu_reduce_update_broadcast(self, layer, peer_grad, world: int, rank: int, peer_w, train_ctx, step: int):
        lin = _optim(train_ctx.optimiser)
        self._check(self.lib.sk_reduce_update_broadcast(self.handle, C.byref(layer.desc()), peer_grad, world, rank,
                                                        peer_w, C.byref(lin), train_ctx.learn_rate, train_ctx.grad_clamp,
                                                        step & 0xFFFFFFFF))

    def peer_alloc(self, nbytes: int):
        """(device pointer, 64-byte IPC handle) of a zeroed exchange arena on this context's device."""
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        self._check(self.lib.sk_peer_alloc(self.handle, nbytes, C.byref(ptr), handle))
        return ptr.value, handle.raw

    def peer_open(self, handle: bytes) -> int:
        ptr = C.c_void_p()
        self._check(self.lib.sk_peer_open(self.handle, handle, C.byref(ptr)))
        return ptr.value

    def peer_close(self, ptr: int):
        self._check(self.lib.sk_peer_close(self.handle, C.c_void_p(ptr)))

    def peer_free(self, ptr: int):
        self._check(self.lib.sk_peer_free(self.handle, C.c_void_p(ptr)))

    def copy_into(self, dst: Tensor, src_ptr: int, nbytes: int):
        """Device-to-device copy on the context's stream (receive buffer -> weight tensor)."""
        self._check(self.lib.sk_copy(self.handle, dst.ptr(), C.c_void_p(src_ptr), nbytes))

    def signal_peers(self, peer_flags, world: int, slot: int, value: int):
        self._check(self.lib.sk_signal_peers(self.handle, peer_flags, world, slot, value & 0xFFFFFFFF))

    def wait_flags(self, flags_ptr: int, world: int, value: int):
        self._check(self.lib.sk_wait_flags(self.handle, C.c_void_p(flags_ptr), world, value & 0xFFFFFFFF))
