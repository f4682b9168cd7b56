"""Data-parallel training of a FeedForwardNetwork: one process per GPU, batch rows split
across ranks, parameters replicated. No counterpart in the reference (single device).

Forward, loss delta and hidden deltas are independent per row; the only exchange is the sum
over rows of dW, dB and the normalisation-parameter gradients. Because every hidden delta
must read the next layer's weights AFTER that layer's update (src/ffn.rs:141-163), the
order per layer is: local batch sums -> all-reduce (NCCL) -> optimiser step -> delta of the
layer below. Dropout hashes the global row index and every 1/M uses the global batch, so N
ranks reproduce the single-device result up to the order of the f32 sums.

Two exchange schemes:

* "allreduce": f32 dW and column sums are all-reduced, every rank runs the whole optimiser step.
* "sharded" (default for 16-bit blocks whose row count divides by the rank count): dW is produced
  in the storage type, already averaged, and reduce-scattered by rows; each rank steps only its
  1/W of the rows (f32 master, moments, 16-bit copy), then the 16-bit weights are all-gathered in
  place. This halves the bytes on NVLink and divides the optimiser's HBM traffic by W. The f32
  master weights and moments of a rank are then current only for the rows it owns
  (`owned_rows(i)`); the 16-bit weights are complete everywhere.

* "fused" (default for 16-bit blocks on up to 8 GPUs of one node): the same sharding, but without
  library collectives on the weight path. Every rank keeps one exchange arena (gradient buffer, weight
  tensor and flag words of every layer) and maps the other ranks' arenas into its address space (CUDA
  IPC). Each rank writes its 16-bit dW into its own gradient buffer; after a flag handshake ONE kernel
  per rank pulls the rows it owns out of all gradient buffers over NVLink, adds them, steps them and
  stores the new 16-bit rows into every rank's weight tensor (reduce-scatter + optimiser + all-gather
  fused); a second handshake releases the dX GEMM below.
  All flag waits are bounded (SK_ERR_DEVICE_TIMEOUT instead of a hang). Only the small column sums
  still use an NCCL all-reduce.

* "native" (default for 16-bit networks without BatchNorm on 2, 4 or 8 GPUs of one node): the fused
  exchange with the whole backward pass sequenced in ONE native call (sk_dp_backward), optionally in P
  blocks of weight rows: per block the dW GEMM writes the local gradient and raises a flag on the other
  ranks, one kernel waits for their flags, sums, steps and redistributes the rows this rank owns, and the dX
  GEMM of the layer below waits inside its TMA producer only for the blocks its tile needs. Column sums
  travel through the same arena; no library collective and no host-side handshake is left on the step. With
  `multicast` the arena lives in torch's symmetric memory and the kernel reduces inside the NVSwitch and
  sends each row once. Inside block c of a matrix with K rows, rank r owns rows
  [c*K/P + r*K/(P*W), c*K/P + (r+1)*K/(P*W)) (`owned_row_ranges(i)`).

Under every sharded scheme a rank's f32 master weights and moments are current only for the rows it owns.
`gather_state()` (collective) makes them complete on every rank; call it before saving a checkpoint or
converting a block, and `close()` calls it.

BatchNorm blocks (hidden ones) run their forward in three phases around two all-reduces of the column
statistics, so that mean and variance are those of the whole batch.

Failure detection: device-side waits are bounded (SK_ERR_DEVICE_TIMEOUT). With `collective_timeout`
(seconds) set, every library collective is waited for on the host with that deadline and a rank that never
joins turns into log.DriverError on the others instead of a hang.
"""
from __future__ import annotations

import ctypes as C
import datetime
from typing import Sequence

import torch
import torch.distributed as dist

from . import log
from .context import LossConfig, MultiLayerTrainContext
from .core import Tensor
from .ffn import FeedForwardNetwork
from .function import Normalisation


class _ArenaView:
    """Exposes a range of an exchange arena through __cuda_array_interface__ (as 16-bit integers)."""

    def __init__(self, ptr: int, count: int):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<i2", "data": (ptr, False), "version": 2}


def _alias_tensor(ptr: int, shape, dtype, device) -> torch.Tensor:
    """A torch tensor of a 16-bit dtype over library-owned device memory (no copy, no ownership)."""
    count = 1
    for d in shape:
        count *= d
    raw = torch.as_tensor(_ArenaView(ptr, count), device=device)
    assert raw.data_ptr() == ptr, "torch copied the arena range instead of aliasing it"
    return raw.view(dtype).view(*shape)


def shard_rows(global_batch: int, rank: int, world: int):
    """(first row, row count) of this rank's contiguous shard; the batch must divide evenly."""
    if global_batch % world != 0:
        raise log.InvalidBatchSize(f"global batch {global_batch} is not divisible by {world} ranks")
    per = global_batch // world
    return rank * per, per


class DataParallelFFN:
    def __init__(self, context, network: FeedForwardNetwork, global_batch: int, rank: int, world: int, group=None,
                 scheme: str = "auto", chunks: int = 0, collective_timeout: float | None = None, multicast=False):
        self.ctx, self.net, self.group = context, network, group
        self.rank, self.world, self.global_batch = rank, world, global_batch
        self.collective_timeout = collective_timeout
        # multicast (True / False / "auto"): put the exchange arena in torch's symmetric memory and, where the node
        # has NVSwitch multicast, let the native exchange reduce inside the switch and send each row once; "auto"
        # falls back to the library's own arenas when symmetric memory cannot be set up. Not for jobs in which a
        # rank may leave while the others keep running.
        self.multicast, self.mc_base, self._symm = multicast, 0, None
        self.native = False
        self.blocks = []
        self.row_offset, self.local_batch = shard_rows(global_batch, rank, world)
        # BatchNorm takes its column statistics over the whole batch: its forward runs in three phases
        # with two small all-reduces (hidden blocks only: the output-layer delta has no global 1/M).
        self.bn_stats = {}
        if world > 1:
            for i, layer in enumerate(network.get_layers()):
                if layer.get_normalisation() == Normalisation.BatchNorm:
                    if i == len(network.get_layers()) - 1:
                        raise log.InvalidConfiguration("BatchNorm on the output block is not supported under data parallelism")
                    self.bn_stats[i] = torch.zeros(2, layer.get_weights().cols(), device=context.device, dtype=torch.float32)
        dev = context.device
        layers = network.get_layers() if world > 1 else []
        self.fused = False
        self.sharded = []
        self.dw, self.dw_shard = [], []
        for l in layers:
            k, n = l.get_weights().rows(), l.get_weights().cols()
            can_shard = getattr(l, "precision", None) is not None and l.precision.value != 0 and k % world == 0
            use = scheme in ("sharded", "fused") or (scheme == "auto" and can_shard)
            if use and not can_shard:
                raise log.InvalidConfiguration("sharded exchange needs 16-bit blocks whose rows divide by the rank count")
            self.sharded.append(use)
            if use:
                dt = l.get_weights().data.dtype
                self.dw.append(torch.empty(k, n, device=dev, dtype=dt))
                self.dw_shard.append(torch.empty(k // world, n, device=dev, dtype=dt))
            else:
                self.dw.append(torch.empty(k, n, device=dev, dtype=torch.float32))
                self.dw_shard.append(None)
        self.colsums = [torch.empty(3, l.get_weights().cols(), device=dev, dtype=torch.float32) for l in layers]
        self.collectives = 0
        want = chunks if chunks > 0 else 1
        can_native = (world in (2, 4, 8) and hasattr(context, "gpu_dp_backward") and not self.bn_stats and bool(layers)
                        and all(getattr(l, "precision", None) is not None and l.precision.value != 0 for l in layers)
                        and all(context.dp_blocks(l.get_weights().rows(), l.get_weights().cols(), world, want) > 0 for l in layers))
        if scheme == "native" and not can_native:
            raise log.InvalidConfiguration("the native exchange needs 2, 4 or 8 ranks and 16-bit blocks without BatchNorm "
                                           "whose rows split evenly")
        self.native = can_native and scheme in ("auto", "native")
        self.fused = not self.native and (scheme == "fused" or (scheme == "auto" and world > 1 and all(self.sharded)
                                                                   and world <= 8 and hasattr(context, "signal_peers")))
        self.epoch = 0
        if world > 1 and hasattr(context, "set_colsum_handover"):
            # backward() calls the delta of a layer and its weight-gradient GEMM back to back
            context.set_colsum_handover(True)
        if self.native:
            self.sharded = [True] * len(layers)
            self.blocks = [context.dp_blocks(l.get_weights().rows(), l.get_weights().cols(), world, want) for l in layers]
            self.want_blocks = want

        if self.fused or self.native:
            self.dw, self.dw_shard = [], []      # these exchanges stage gradients in their own arena
            self._map_peers(layers)

    def _map_peers(self, layers):
        """One exchange arena per rank (staging buffer, receive buffer and flag words of every layer),
        allocated by the library, exported as a CUDA IPC handle and mapped by every other rank with its
        own device current. Keeps pointer tables: staging / receive / flags of every rank per layer."""
        W, es = self.world, layers[0].get_weights().data.element_size()
        flag_bytes = max(256, self.ctx.dp_flag_bytes() if hasattr(self.ctx, "dp_flag_bytes") else 256)
        offsets, total = [], 0
        for l in layers:
            nbytes = l.get_weights().rows() * l.get_weights().cols() * es
            pad = lambda v: (v + 255) // 256 * 256
            off_stage = total
            off_recv = off_stage + pad(nbytes)
            off_flags = off_recv + pad(nbytes)
            off_colsums = off_flags + pad(flag_bytes)
            total = off_colsums + pad(3 * l.get_weights().cols() * 4)
            offsets.append((off_stage, off_recv, off_flags, nbytes, off_colsums))
        symm = None
        if self.multicast:
            # torch's symmetric memory: one allocation per rank, mapped into every rank and bound to a multicast object
            try:
                import torch.distributed._symmetric_memory as symm_mem
                buf = symm_mem.empty(total, dtype=torch.uint8, device=self.ctx.device)
                hdl = symm_mem.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
                symm = (buf, hdl)
            except Exception:
                if self.multicast != "auto":
                    raise
            # every rank must take the same road
            ok = torch.tensor([1 if symm is not None else 0], device=self.ctx.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
            if int(ok.item()) == 0:
                symm = None
        if symm is not None:
            buf, hdl = symm
            buf.zero_()
            self._symm = symm
            self._arena = buf.data_ptr()
            self._bases = [int(p) for p in hdl.buffer_ptrs]
            assert self._bases[self.rank] == self._arena, "symmetric memory: this rank's entry is not its own buffer"
            self.mc_base = int(hdl.multicast_ptr) if hdl.multicast_ptr else 0
        else:
            self._arena, handle = self.ctx.peer_alloc(total)
            table = [None] * W
            dist.all_gather_object(table, handle, group=self.group)
            self._bases = [self._arena if r == self.rank else self.ctx.peer_open(table[r]) for r in range(W)]
        self._offsets = offsets
        arr = lambda off: (C.c_void_p * W)(*[b + off for b in self._bases])
        self.stage_ptr, self.recv_ptr, self.flag_ptr, self.nbytes = [], [], [], []
        self.p_stage, self.p_recv, self.p_flag_a, self.p_flag_b, self.p_colsums = [], [], [], [], []
        for off_stage, off_recv, off_flags, nbytes, off_colsums in offsets:
            self.stage_ptr.append(self._arena + off_stage)
            self.recv_ptr.append(self._arena + off_recv)
            self.flag_ptr.append(self._arena + off_flags)
            self.nbytes.append(nbytes)
            self.p_stage.append(arr(off_stage))
            self.p_recv.append(arr(off_recv))
            self.p_flag_a.append(arr(off_flags))
            self.p_flag_b.append(arr(off_flags + 4 * W))
            self.p_colsums.append(arr(off_colsums))
        # The receive buffer of a layer becomes the storage of its weight tensor: the owners' stores land
        # directly in every rank's weights and no copy is needed after the second handshake.
        self._own_w = []
        for l, rp in zip(layers, self.recv_ptr):
            w = l.get_weights()
            self._own_w.append(w.data)
            alias = _alias_tensor(rp, tuple(w.data.shape), w.data.dtype, self.ctx.device)
            alias.copy_(w.data)
            w.data = alias
            l._desc = None
        torch.cuda.synchronize(self.ctx.device)
        dist.barrier(group=self.group)

    def exchange_name(self) -> str:
        if self.world == 1:
            return "none"
        if self.native:
            return "native+multicast" if self.mc_base else "native"
        return "fused" if self.fused else "nccl"

    def _collective(self, fn, *args, **kwargs):
        """A library collective on the context's stream; with `collective_timeout` set it is waited for on
        the host and a rank that never joins becomes an error on the others."""
        self.collectives += 1
        if self.collective_timeout is None:
            stream = getattr(self.ctx, "stream", None)
            if stream is not None and self.ctx.device.type == "cuda":
                with torch.cuda.stream(stream):   # the kernels around it run on this stream, not torch's current one
                    return fn(*args, group=self.group, **kwargs)
            return fn(*args, group=self.group, **kwargs)
        work = fn(*args, group=self.group, async_op=True, **kwargs)
        try:
            done = work.wait(timeout=datetime.timedelta(seconds=self.collective_timeout))
        except RuntimeError as e:
            raise log.DriverError(f"collective did not complete within {self.collective_timeout} s: {e}") from e
        if done is False:
            raise log.DriverError(f"collective did not complete within {self.collective_timeout} s: a rank did not join")

    def owned_row_ranges(self, i: int):
        """[(first row, row count), ...] of layer i's weight matrix whose f32 masters and moments this rank keeps current."""
        k = self.net.get_layers()[i].get_weights().rows()
        if self.world > 1 and self.native:
            p = self.blocks[i]
            own = k // (p * self.world)
            return [(c * (k // p) + self.rank * own, own) for c in range(p)]
        return [self.owned_rows(i)]

    def gather_state(self):
        """Collective: complete the f32 master weights and both moments of every sharded layer on every rank
        (each rank contributes the rows it owns). After it, checkpoints and precision conversions see current
        state everywhere (the contract of src/io/save.rs:227-346)."""
        if self.world == 1:
            return
        if hasattr(self.ctx, "synchronize"):
            self.ctx.synchronize()
        for i, layer in enumerate(self.net.get_layers()):
            if not self.sharded[i]:
                continue
            p = self.blocks[i] if self.native else 1
            for t in (layer.get_master_weights(), layer.get_dv_weights(), layer.get_dm_weights()):
                if t is None:
                    continue
                k, n = t.data.shape
                own = k // (p * self.world)
                view = t.data.view(p, self.world, own * n)
                mine = view[:, self.rank].contiguous()
                parts = [torch.empty_like(mine) for _ in range(self.world)]
                self._collective(dist.all_gather, parts, mine)
                for r, part in enumerate(parts):
                    view[:, r].copy_(part)

    def close(self):
        """Complete the sharded optimiser state, unmap the other ranks' arenas and free this rank's
        (collective: every rank calls it)."""
        if self.world > 1 and any(self.sharded) and getattr(self, "_closed", False) is False:
            self.gather_state()
            self._closed = True
        if getattr(self, "_bases", None):
            torch.cuda.synchronize(self.ctx.device)
            dist.barrier(group=self.group)
            for l, own in zip(self.net.get_layers(), self._own_w):   # weights move back to their own storage
                own.copy_(l.get_weights().data)
                l.get_weights().data = own
                l._desc = None
            torch.cuda.synchronize(self.ctx.device)
            if self._symm is None:
                for r, b in enumerate(self._bases):
                    if r != self.rank:
                        self.ctx.peer_close(b)
                dist.barrier(group=self.group)
                self.ctx.peer_free(self._arena)
            else:
                dist.barrier(group=self.group)
                self._symm = None
            self._bases = None

    def owned_rows(self, i: int):
        """(first row, row count) of layer i's weight matrix whose master weights and moments this rank keeps current."""
        k = self.net.get_layers()[i].get_weights().rows()
        if self.world > 1 and self.sharded[i]:
            return self.rank * (k // self.world), k // self.world
        return 0, k

    def forward(self, input: Tensor, use_dropout: bool, step: int):
        if not self.bn_stats:
            return self.net.forward(self.ctx, input, self.local_batch, use_dropout, step, self.row_offset)
        outputs, cur = [], input
        for i, layer in enumerate(self.net.get_layers()):
            stats = self.bn_stats.get(i)
            if stats is None:
                cur = layer.forward(self.ctx, cur, self.local_batch, use_dropout, step, self.row_offset)
            else:
                layer.check_input_dimension(cur, self.local_batch)
                for phase in (0, 1, 2):
                    self.ctx.gpu_forward_batchnorm_phase(layer, cur, self.local_batch, self.global_batch, phase, stats,
                                                         use_dropout, step, self.row_offset)
                    if phase < 2:
                        self._collective(dist.all_reduce, stats[phase])
                cur = layer.get_outputs()
            outputs.append(cur)
        return outputs

    def _exchange(self, i: int):
        if self.world > 1:
            self._collective(dist.all_reduce, self.dw[i])
            self._collective(dist.all_reduce, self.colsums[i])

    def backward(self, outputs: Sequence[Tensor], target: Tensor, input: Tensor, loss_config: LossConfig,
                 train_ctx: MultiLayerTrainContext, step: int):
        layers = self.net.get_layers()
        n = len(layers)
        if len(outputs) != n or len(train_ctx.optimisers) != n:
            raise log.InvalidConfiguration(f"Backward pass expects exactly {n} activation vectors and optimizers.")
        if train_ctx.batch_size != self.global_batch:
            raise log.InvalidBatchSize("train context batch size must be the global batch")
        if self.world == 1:   # nothing to exchange: the plain reference-order backward
            self.net.backward(self.ctx, outputs, target, input, loss_config, train_ctx, step)
            return
        last = n - 1
        self.epoch += 1
        if self.native:
            self.net._check_backward(target, input, loss_config, _LocalBatch(train_ctx, self.local_batch))
            self.ctx.gpu_dp_backward(layers, self._exchange_tables(), target, input, loss_config, train_ctx, self.local_batch,
                                     self.global_batch, self.world, self.rank, self.want_blocks, self.epoch, step)
            return
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
            tci = train_ctx.get_train_context(i)
            if self.fused:
                W, e = self.world, self.epoch
                self.ctx.gpu_backward_grads_lp(layer, x, self.local_batch, self.global_batch, self.stage_ptr[i],
                                               self.colsums[i])                 # dW into my arena's gradient buffer
                self.ctx.signal_peers(self.p_flag_a[i], W, self.rank, e)       # my gradient buffer is complete
                self._collective(dist.all_reduce, self.colsums[i])
                self.ctx.wait_flags(self.flag_ptr[i], W, e)                     # so is everybody else's
                self.ctx.gpu_reduce_update_broadcast(layer, self.p_stage[i], W, self.rank, self.p_recv[i], tci, step)
                self.ctx.signal_peers(self.p_flag_b[i], W, self.rank, e)       # my rows are in every weight tensor
                self.ctx.gpu_apply_vector_update(layer, self.colsums[i], self.global_batch, tci, step)
                self.ctx.wait_flags(self.flag_ptr[i] + 4 * W, W, e)             # all rows of this layer have arrived
                continue
            if self.sharded[i]:
                self.ctx.gpu_backward_grads_lp(layer, x, self.local_batch, self.global_batch, self.dw[i], self.colsums[i])
                self._collective(dist.reduce_scatter_tensor, self.dw_shard[i], self.dw[i])
                self._collective(dist.all_reduce, self.colsums[i])
                row0, nrows = self.owned_rows(i)
                self.ctx.gpu_apply_update_rows(layer, self.dw_shard[i], row0, nrows, tci, step)
                self.ctx.gpu_apply_vector_update(layer, self.colsums[i], self.global_batch, tci, step)
                w = layer.get_weights().data
                self._collective(dist.all_gather_into_tensor, w, w[row0:row0 + nrows])
                continue
            self.ctx.gpu_backward_grads(layer, x, self.local_batch, self.dw[i], self.colsums[i])
            self._exchange(i)
            self.ctx.gpu_apply_update(layer, self.dw[i], self.colsums[i], self.global_batch, tci, step)

    def _exchange_tables(self):
        """Per layer the four pointer tables sk_dp_backward takes (built once)."""
        if getattr(self, "_tables", None) is None:
            from ._native import SkExchange
            n = len(self.p_stage)
            tabs = (SkExchange * n)()
            for i in range(n):
                tabs[i].peer_grad = C.cast(self.p_stage[i], C.c_void_p)
                tabs[i].peer_w = C.cast(self.p_recv[i], C.c_void_p)
                tabs[i].peer_flags = C.cast(self.p_flag_a[i], C.c_void_p)
                tabs[i].peer_colsums = C.cast(self.p_colsums[i], C.c_void_p)
                if self.mc_base:
                    off_stage, off_recv = self._offsets[i][0], self._offsets[i][1]
                    tabs[i].mc_grad, tabs[i].mc_w = self.mc_base + off_stage, self.mc_base + off_recv
            self._tables = tabs
        return self._tables


class _LocalBatch:
    """A MultiLayerTrainContext seen with this rank's row count (for the host-side shape checks)."""

    def __init__(self, train_ctx, local_batch):
        self.batch_size, self.optimisers = local_batch, train_ctx.optimisers
