"""Host logic of data-parallel training on two CPU ranks (gloo): row sharding, the order of
gradient exchange / update / hidden delta, and that both ranks apply the same summed gradient.
The device calls are replaced by a recording fake; the kernels themselves are covered on a GPU."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _T:
    def __init__(self, r, c):
        self._r, self._c = r, c

    def rows(self):
        return self._r

    def cols(self):
        return self._c


class _Layer:
    def __init__(self, k, n, idx, log):
        from soklyn_b200.function import Normalisation
        self.k, self.n, self.idx, self.log = k, n, idx, log
        self.norm = Normalisation.Disabled

    def get_weights(self):
        return _T(self.k, self.n)

    def get_normalisation(self):
        return self.norm

    def forward(self, ctx, x, batch, use_dropout, step, row_offset=0):
        self.log.append(("forward", self.idx, batch, row_offset))
        return _T(batch, self.n)

    def compute_loss(self, ctx, target, loss_config):
        self.log.append(("loss", self.idx))


class _Ctx:
    """Stands in for GpuContext: rank r contributes (r+1)*(layer+1) to every gradient element."""

    def __init__(self, rank, log):
        self.device, self.rank, self.log = torch.device("cpu"), rank, log
        self.applied = {}

    def gpu_hidden_layer_error(self, cur, nxt, batch, batch_stat):
        self.log.append(("hidden", cur.idx, nxt.idx, batch, batch_stat))

    def gpu_backward_grads(self, layer, x, batch, dw, colsums):
        self.log.append(("grads", layer.idx, batch))
        dw.fill_((self.rank + 1) * (layer.idx + 1))
        colsums.fill_(10.0 * (self.rank + 1))

    def gpu_apply_update(self, layer, dw, colsums, batch_stat, train_ctx, step):
        self.log.append(("apply", layer.idx, batch_stat))
        self.applied[layer.idx] = (float(dw[0, 0]), float(dw.min()), float(dw.max()), float(colsums[2, -1]))

    def gpu_backward_pass(self, layer, x, train_ctx, step):
        self.log.append(("fused", layer.idx))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from soklyn_b200.context import LossConfig, MultiLayerTrainContext
    from soklyn_b200.dp import DataParallelFFN
    from soklyn_b200.ffn import FeedForwardNetwork
    from soklyn_b200.function import Activation, LossFunc, Optimiser
    log = []
    layers = [_Layer(6, 5, 0, log), _Layer(5, 4, 1, log), _Layer(4, 3, 2, log)]
    ctx = _Ctx(rank, log)
    dp = DataParallelFFN(ctx, FeedForwardNetwork(layers, 6), global_batch=8, rank=rank, world=world)
    outs = dp.forward(_T(4, 6), False, 1)
    opt = [Optimiser.Adam()] * 3
    dp.backward(outs, _T(4, 3), _T(4, 6), LossConfig(LossFunc.MeanSquareLoss, Activation.Identity),
                MultiLayerTrainContext(opt, opt, 8, 1e-3), 1)
    q.put((rank, log, ctx.applied, dp.row_offset, dp.local_batch, dp.collectives))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_exchange_and_ordering():
    world, port = 2, 29000 + os.getpid() % 2000
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    procs = [ctxm.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, log, applied, row_offset, local, collectives in results:
        assert (row_offset, local) == (4 * rank, 4)
        assert collectives == 6                                # dW + column sums per layer
        assert [e for e in log if e[0] == "forward"] == [("forward", i, 4, 4 * rank) for i in range(3)]
        for i in range(3):                                      # sum over ranks: (1 + 2) * (layer + 1)
            first, lo, hi, cs = applied[i]
            assert first == lo == hi == 3.0 * (i + 1) and cs == 30.0
        order = [e[:2] for e in log if e[0] in ("loss", "hidden", "grads", "apply")]
        assert order == [("loss", 2), ("grads", 2), ("apply", 2), ("hidden", 1), ("grads", 1), ("apply", 1),
                         ("hidden", 0), ("grads", 0), ("apply", 0)]
        assert all(e[3:] == (4, 8) for e in log if e[0] == "hidden")      # local rows, global 1/M
        assert all(e[2] == 8 for e in log if e[0] == "apply")
    assert results[0][2] == results[1][2]                       # both ranks step with identical gradients


def test_shard_rows_and_single_rank_path():
    sys.path.insert(0, ROOT)
    from soklyn_b200 import log as sklog
    from soklyn_b200.dp import shard_rows
    assert shard_rows(8192, 3, 8) == (3072, 1024)
    assert shard_rows(10, 0, 1) == (0, 10)
    with pytest.raises(sklog.InvalidBatchSize):
        shard_rows(10, 0, 4)


def _bn_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from soklyn_b200.dp import DataParallelFFN
    from soklyn_b200.ffn import FeedForwardNetwork
    from soklyn_b200.function import Normalisation
    log = []

    class BnLayer(_Layer):
        def check_input_dimension(self, x, batch):
            log.append(("check", self.idx, x.rows(), batch))

        def get_outputs(self):
            return _T(4, self.n)

    class BnCtx(_Ctx):
        def gpu_forward_batchnorm_phase(self, layer, x, batch, batch_stat, phase, stats, use_dropout, step, row_offset=0):
            if phase < 2:
                stats[phase].fill_(float((self.rank + 1) * (phase + 1)))     # this shard's partial sums
            log.append(("bn", layer.idx, phase, batch, batch_stat, row_offset, stats.clone().tolist()))

    layers = [BnLayer(6, 5, 0, log), _Layer(5, 3, 1, log)]
    layers[0].norm = Normalisation.BatchNorm
    dp = DataParallelFFN(BnCtx(rank, log), FeedForwardNetwork(layers, 6), global_batch=8, rank=rank, world=world)
    outs = dp.forward(_T(4, 6), True, 3)
    q.put((rank, log, len(outs), dp.collectives))
    dist.barrier()
    dist.destroy_process_group()


def test_batchnorm_forward_sums_statistics_over_ranks_between_phases():
    world, port = 2, 31000 + os.getpid() % 2000
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    procs = [ctxm.Process(target=_bn_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, log, n_outs, collectives in results:
        assert n_outs == 2 and collectives == 2
        bn = [e for e in log if e[0] == "bn"]
        assert [e[2] for e in bn] == [0, 1, 2] and all(e[3:6] == (4, 8, 4 * rank) for e in bn)
        # phase 1 sees the column sums of both ranks (1 + 2), phase 2 also the summed squares (2 + 4)
        assert bn[1][6][0] == [3.0] * 5
        assert bn[2][6] == [[3.0] * 5, [6.0] * 5]
        assert ("forward", 1, 4, 4 * rank) in log                 # the block after it runs the ordinary forward


def test_batchnorm_output_block_is_rejected_under_data_parallelism():
    sys.path.insert(0, ROOT)
    from soklyn_b200 import log as sklog
    from soklyn_b200.dp import DataParallelFFN
    from soklyn_b200.ffn import FeedForwardNetwork
    from soklyn_b200.function import Normalisation
    layers = [_Layer(6, 5, 0, []), _Layer(5, 3, 1, [])]
    layers[1].norm = Normalisation.BatchNorm
    with pytest.raises(sklog.InvalidConfiguration):
        DataParallelFFN(_Ctx(0, []), FeedForwardNetwork(layers, 6), global_batch=8, rank=0, world=2, scheme="allreduce")


class _Data(_T):
    """A fake tensor that also carries storage (what gather_state and the sharded schemes touch)."""

    def __init__(self, data):
        super().__init__(*data.shape)
        self.data = data


class _ShardedLayer(_Layer):
    """16-bit block whose f32 masters and moments start as zeros; a rank marks the rows it owns."""

    def __init__(self, k, n, idx, log):
        super().__init__(k, n, idx, log)
        from soklyn_b200.function import Precision
        self.precision = Precision.FP16
        self.w = _Data(torch.zeros(k, n, dtype=torch.float16))
        self.master, self.dv, self.dm = (_Data(torch.zeros(k, n)) for _ in range(3))

    def get_weights(self):
        return self.w

    def get_master_weights(self):
        return self.master

    def get_dv_weights(self):
        return self.dv

    def get_dm_weights(self):
        return self.dm


def _gather_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from soklyn_b200.dp import DataParallelFFN
    from soklyn_b200.ffn import FeedForwardNetwork
    layers = [_ShardedLayer(8, 3, 0, []), _ShardedLayer(4, 5, 1, [])]
    dp = DataParallelFFN(_Ctx(rank, []), FeedForwardNetwork(layers, 8), global_batch=8, rank=rank, world=world, scheme="sharded")
    # pretend two blocks of rows per matrix, as the native exchange lays them out
    dp.native, dp.blocks = True, [2, 1]
    for i, layer in enumerate(layers):
        for first, count in dp.owned_row_ranges(i):
            for t, scale in ((layer.master, 1.0), (layer.dv, 10.0), (layer.dm, 100.0)):
                t.data[first:first + count] = scale * (rank + 1) + torch.arange(first, first + count).float().unsqueeze(1) / 100
    ranges = [dp.owned_row_ranges(i) for i in range(2)]
    dp.gather_state()
    q.put((rank, ranges, [(l.master.data.clone(), l.dv.data.clone(), l.dm.data.clone()) for l in layers]))
    dist.barrier()
    dist.destroy_process_group()


def test_gather_state_completes_sharded_masters_and_moments_on_every_rank():
    world, port = 2, 33000 + os.getpid() % 2000
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    procs = [ctxm.Process(target=_gather_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, ranges0, state0), (_, ranges1, state1) = results
    assert ranges0 == [[(0, 2), (4, 2)], [(0, 2)]] and ranges1 == [[(2, 2), (6, 2)], [(2, 2)]]
    for (m0, v0, d0), (m1, v1, d1), k in zip(state0, state1, (8, 4)):
        assert torch.equal(m0, m1) and torch.equal(v0, v1) and torch.equal(d0, d1)     # complete and identical
        owner = torch.tensor([(1 if any(f <= r < f + c for f, c in rr) else 2)
                              for r in range(k) for rr in [ranges0[0] if k == 8 else ranges0[1]]]).float()
        rows = torch.arange(k).float() / 100
        assert torch.allclose(m0[:, 0], owner + rows) and torch.allclose(v0[:, 0], 10 * owner + rows)
        assert torch.allclose(d0[:, 0], 100 * owner + rows)


def _absent_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from soklyn_b200 import log as sklog
    from soklyn_b200.context import LossConfig, MultiLayerTrainContext
    from soklyn_b200.dp import DataParallelFFN
    from soklyn_b200.ffn import FeedForwardNetwork
    from soklyn_b200.function import Activation, LossFunc, Optimiser
    log = []
    layers = [_Layer(6, 5, 0, log), _Layer(5, 3, 1, log)]
    dp = DataParallelFFN(_Ctx(rank, log), FeedForwardNetwork(layers, 6), global_batch=8, rank=rank, world=world,
                         collective_timeout=2.0)
    outs = dp.forward(_T(4, 6), False, 1)
    opt = [Optimiser.Adam()] * 2
    outcome = "skipped"
    if rank == 0:       # rank 1 fails on the host before its first collective and never joins it
        try:
            dp.backward(outs, _T(4, 3), _T(4, 6), LossConfig(LossFunc.MeanSquareLoss, Activation.Identity),
                        MultiLayerTrainContext(opt, opt, 8, 1e-3), 1)
            outcome = "completed"
        except sklog.DriverError as e:
            outcome = "error: " + str(e)[:60]
    q.put((rank, outcome, [e[0] for e in log]))
    import time
    time.sleep(0.5 if rank == 0 else 4.0)   # the absent rank stays alive past the other's deadline
    os._exit(0)                             # no collective teardown: the group is broken by design


def test_rank_that_never_joins_a_collective_becomes_an_error_after_the_host_deadline():
    """Failure made on the host, no GPU involved: rank 1 skips its backward pass; rank 0's first gradient
    all-reduce has nobody to meet and must end in an error status within the deadline, not hang."""
    import time
    world, port = 2, 35000 + os.getpid() % 2000
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    procs = [ctxm.Process(target=_absent_worker, args=(r, world, port, q)) for r in range(world)]
    t0 = time.time()
    for p in procs:
        p.start()
    results = dict((r, (o, l)) for r, o, l in (q.get(timeout=60) for _ in range(world)))
    assert time.time() - t0 < 45
    for p in procs:
        p.join(timeout=30)
    assert results[1][0] == "skipped"
    assert results[0][0].startswith("error: collective did not complete"), results[0]
    assert "apply" not in results[0][1]          # nothing was stepped with a partial sum
