"""Error behaviour of the drop-in API (the checks of src/mlp.rs and src/io/device.rs), status codes
of the C ABI called directly, checkpoint round trip, and the utility kernels."""
import ctypes as C
import os

import numpy as np
import pytest

import harness as H
import soklyn_b200 as sk
from soklyn_b200 import _native, configs, log
from soklyn_b200.configs import _GivenWeights

pytestmark = pytest.mark.gpu


def _block(ctx, k=12, n=8, batch=6, training=True, prec=sk.Precision.FP32, cfg=None):
    w = np.random.default_rng(3).standard_normal((k, n)).astype(np.float32) * 0.1
    return sk.DenseBlock(ctx, training, k, n, batch, _GivenWeights(w), cfg or sk.LayerInitConfig(), prec)


def _x(ctx, rows, cols, prec=sk.Precision.FP32):
    return sk.Tensor.from_cpu_vector(ctx, np.ones((rows, cols), np.float32), (rows, cols), prec)


def test_constructor_and_forward_checks(gpu_ctx):
    with pytest.raises(log.InvalidConfiguration):
        sk.DenseBlock(gpu_ctx, True, 0, 4, 4, sk.InitZeroFunc())
    with pytest.raises(log.InvalidConfiguration):
        sk.DenseBlock(gpu_ctx, True, 4, 4, 0, sk.InitZeroFunc())
    blk = _block(gpu_ctx)
    with pytest.raises(log.MismatchedDimensions):
        blk.forward(gpu_ctx, _x(gpu_ctx, 4, 12), 5, False, 1)           # fewer rows than the batch
    with pytest.raises(log.AllocationLimitExceeded):
        blk.forward(gpu_ctx, _x(gpu_ctx, 7, 12), 6, False, 1)           # more rows than max_batch
    with pytest.raises(log.MismatchedDimensions):
        blk.forward(gpu_ctx, _x(gpu_ctx, 6, 11), 6, False, 1)           # wrong feature count
    with pytest.raises(log.InvalidBatchSize):
        blk.forward(gpu_ctx, _x(gpu_ctx, 6, 12), 0, False, 1)
    blk.set_activation(sk.Activation.Softmax)
    with pytest.raises(log.InvalidConfiguration):
        blk.forward(gpu_ctx, _x(gpu_ctx, 6, 12), 6, False, 1)
    blk.set_activation(sk.Activation.ReLU)
    blk.set_normalisation(sk.Normalisation.BatchNorm)
    with pytest.raises(log.InvalidBatchSize):
        blk.forward(gpu_ctx, _x(gpu_ctx, 6, 12), 1, False, 1)
    assert blk.forward(gpu_ctx, _x(gpu_ctx, 6, 12), 6, False, 1) is blk.get_outputs()


def test_backward_and_loss_checks(gpu_ctx):
    inf = _block(gpu_ctx, training=False)
    tc = sk.TrainContext(sk.Optimiser.SGD(), sk.Optimiser.SGD(), 6, 0.1)
    with pytest.raises(log.TrainingModeRequired):
        inf.backward_output(gpu_ctx, _x(gpu_ctx, 6, 12), tc, 1)
    with pytest.raises(log.TrainingModeRequired):
        inf.compute_loss(gpu_ctx, _x(gpu_ctx, 6, 8), sk.LossConfig(sk.LossFunc.MeanSquareLoss, sk.Activation.Identity))
    blk = _block(gpu_ctx)
    with pytest.raises(log.MismatchedDimensions):
        blk.compute_loss(gpu_ctx, _x(gpu_ctx, 6, 7), sk.LossConfig(sk.LossFunc.MeanSquareLoss, sk.Activation.Identity))
    with pytest.raises(log.AllocationLimitExceeded):
        blk.compute_loss(gpu_ctx, _x(gpu_ctx, 9, 8), sk.LossConfig(sk.LossFunc.MeanSquareLoss, sk.Activation.Identity))
    for lf, act in ((sk.LossFunc.MeanSquareLoss, sk.Activation.Softmax), (sk.LossFunc.CrossEntropyLoss, sk.Activation.Sigmoid),
                    (sk.LossFunc.BinaryCrossEntropy, sk.Activation.Softmax)):
        with pytest.raises(log.InvalidConfiguration):
            blk.compute_loss(gpu_ctx, _x(gpu_ctx, 6, 8), sk.LossConfig(lf, act))
    nxt = _block(gpu_ctx, k=9, n=4)                                       # 9 rows do not follow 8 columns
    with pytest.raises(log.MismatchedDimensions):
        blk.backward_hidden(gpu_ctx, nxt, _x(gpu_ctx, 6, 12), tc, 1)
    net = sk.FeedForwardNetwork([blk], 12)
    with pytest.raises(log.InvalidConfiguration):
        net.backward(gpu_ctx, [], _x(gpu_ctx, 6, 8), _x(gpu_ctx, 6, 12),
                     sk.LossConfig(sk.LossFunc.MeanSquareLoss, sk.Activation.Identity),
                     sk.MultiLayerTrainContext([sk.Optimiser.SGD()], [sk.Optimiser.SGD()], 6, 0.1), 1)
    with pytest.raises(log.InvalidConfiguration):
        sk.FeedForwardNetwork([], 12).forward_raw(gpu_ctx, np.zeros(12, np.float32), 1, False, 1)


def test_sixteen_bit_needs_tile_dim_16():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    ctx32 = sk.GpuContext(32, 0)
    try:
        blk = _block(ctx32, prec=sk.Precision.FP16)
        with pytest.raises(log.HardwareConstraintViolation):
            blk.forward(ctx32, _x(ctx32, 6, 12, sk.Precision.FP16), 6, False, 1)
        f32 = _block(ctx32)
        f32.forward(ctx32, _x(ctx32, 6, 12), 6, False, 1)               # f32 accepts tile 32
    finally:
        ctx32.close()


def test_c_abi_status_codes(gpu_ctx):
    lib = _native.lib()
    blk = _block(gpu_ctx)
    d = blk.desc()
    x = _x(gpu_ctx, 6, 12)
    h = gpu_ctx.handle
    assert lib.sk_dense_forward(h, C.byref(d), x.ptr(), 6, 6, 0, 1, 0) == 0
    assert lib.sk_dense_forward(h, C.byref(d), x.ptr(), 4, 6, 0, 1, 0) == 2      # MismatchedDimensions
    assert lib.sk_dense_forward(h, C.byref(d), x.ptr(), 7, 6, 0, 1, 0) == 3      # AllocationLimitExceeded
    assert lib.sk_dense_forward(h, C.byref(d), x.ptr(), 6, 0, 0, 1, 0) == 5      # InvalidBatchSize
    assert lib.sk_dense_forward(h, C.byref(d), None, 6, 6, 0, 1, 0) == 9         # NULL input
    assert b"Batch size" in lib.sk_last_error(h) or b"NULL" in lib.sk_last_error(h)
    bad = type(d)()
    C.memmove(C.byref(bad), C.byref(d), C.sizeof(d))
    bad.act = 5
    assert lib.sk_dense_forward(h, C.byref(bad), x.ptr(), 6, 6, 0, 1, 0) == 4    # Softmax in forward
    bad.act, bad.is_training = 0, 0
    lin = _native.SkOptim(0, 0.0, 0.0, 0.0, 0)
    assert lib.sk_backward_update(h, C.byref(bad), x.ptr(), 6, 6, C.byref(lin), C.byref(lin), 0.1, 1.0, 1) == 6
    assert lib.sk_cast(h, x.ptr(), 0, x.ptr(), 0, 4) == 8                        # f32 -> f32 is not a cast
    assert lib.sk_sync(h) == 0


def test_checkpoint_round_trip(gpu_ctx, tmp_path):
    from soklyn_b200.safetensor import SafetensorFile
    spec = configs.scaled(configs.CONFIGS[4], dims=(64, 128, 64), batch=32, name="ckpt_f16")
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    net, _ = H.run_device(gpu_ctx, spec, w, x, t, 2)
    f = SafetensorFile.from_ffn(gpu_ctx, net)
    f.pass_metadata("epoch", 2)
    path = os.path.join(tmp_path, "net.safetensors")
    f.save(path)
    back = SafetensorFile.read(path)
    assert back.get_metadata() == {"epoch": "2"}
    blocks = back.into_blocks(gpu_ctx, True, 32, sk.Precision.FP16)
    assert len(blocks) == 2
    for a, b in zip(net.get_layers(), blocks):
        for getter in ("get_weights", "get_biases", "get_norm_weights", "get_master_weights", "get_dv_weights",
                       "get_dm_weights", "get_dm_biases", "get_master_norm_weights"):
            assert np.array_equal(getattr(a, getter)().download(gpu_ctx), getattr(b, getter)().download(gpu_ctx)), getter
        assert b.get_normalisation() == sk.Normalisation.Disabled and b.get_activation() == sk.Activation.Identity
    # a resumed network continues exactly like the original once its configuration is set again
    for i, b in enumerate(blocks):
        c = spec.layer_config(i)
        b.set_normalisation(c.normalisation); b.set_activation(c.activation); b.set_mask_coeff(c.mask_coeff)
    resumed = sk.FeedForwardNetwork(blocks, spec.dims[0])
    xd = sk.Tensor.from_cpu_vector(gpu_ctx, x, x.shape, spec.prec())
    o1 = net.forward(gpu_ctx, xd, spec.batch, False, 3)[-1].download(gpu_ctx)
    o2 = resumed.forward(gpu_ctx, xd, spec.batch, False, 3)[-1].download(gpu_ctx)
    assert np.array_equal(o1, o2)
    inference = SafetensorFile.read(path).into_blocks(gpu_ctx, False, 32, sk.Precision.FP16)
    assert inference[0].get_dv_weights() is None and not inference[0].is_training_mode()


def test_cast_fill_and_reset_mask(gpu_ctx):
    a = sk.Tensor.from_cpu_vector(gpu_ctx, np.linspace(-3, 3, 1001, dtype=np.float32), (1001,))
    h = a.cast(gpu_ctx, sk.Precision.FP16)
    assert np.array_equal(h.download(gpu_ctx), np.linspace(-3, 3, 1001, dtype=np.float32).astype(np.float16))
    back = h.cast(gpu_ctx, sk.Precision.FP32)
    assert np.array_equal(back.download(gpu_ctx), h.download(gpu_ctx).astype(np.float32))
    with pytest.raises(log.UnsupportedTypeCast):
        gpu_ctx.gpu_cast_t(a, back)
    blk = _block(gpu_ctx, cfg=sk.LayerInitConfig(sk.Normalisation.Disabled, sk.Activation.ReLU, sk.Regularisation.none(), 0.5))
    blk.forward(gpu_ctx, _x(gpu_ctx, 6, 12), 6, True, 1)
    m = blk.get_masks().download(gpu_ctx)
    assert set(np.unique(m)) <= {0.0, 2.0} and (m == 0).any()
    blk.forward(gpu_ctx, _x(gpu_ctx, 6, 12), 6, False, 2)               # mask persists without dropout
    assert np.array_equal(blk.get_masks().download(gpu_ctx), m)
    blk.reset_mask(gpu_ctx)
    assert (blk.get_masks().download(gpu_ctx) == 1).all()


@pytest.mark.parametrize("prec", ["f16", "bf16"])
def test_batchnorm_and_regularisation_sixteen_bit(gpu_ctx, prec):
    """BatchNorm statistics, L2 regularisation and SGD-Nesterov through the 16-bit path against the f32 oracle."""
    spec = configs.NetSpec(7, "bn_" + prec, (64, 96, 32), ("batch", "disabled"), ("tanh", "identity"), (0.0, 0.0), prec,
                           "mse", "identity", "sgd", 0.05, 48, "xavier_normal", "normal", "normal")
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    if prec == "bf16":
        import torch
        rb = lambda a: torch.from_numpy(a).to(torch.bfloat16).float().numpy()
        w, x, t = [rb(a) for a in w], rb(x), rb(t)
    onet, oloss = H.run_oracle(spec, w, x, t, 1)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 1)
    tol = 1e-2 if prec == "f16" else 6e-2      # bf16 keeps 8 significant bits
    H.compare_states(gpu_ctx, spec, dnet, onet, tol, skip=("mask",))
    np.testing.assert_allclose(dloss, oloss, rtol=tol)


def test_flag_wait_times_out_with_a_status_instead_of_hanging(gpu_ctx):
    """Failure detection of the fused exchange, without faulting anything: wait on flag words that no
    rank ever sets. The kernel gives up after its bound (about two seconds), the next synchronize
    reports SK_ERR_DEVICE_TIMEOUT, and the context stays usable."""
    import time
    import torch
    flags = torch.zeros(4, dtype=torch.int32, device=gpu_ctx.device)
    t0 = time.time()
    gpu_ctx.wait_flags(flags.data_ptr(), 2, 1)
    with pytest.raises(log.NativeError) as e:
        gpu_ctx.synchronize()
    assert "status 11" in str(e.value) and time.time() - t0 < 30
    gpu_ctx.synchronize()                                   # the error word was cleared
    flags.fill_(7)
    gpu_ctx.wait_flags(flags.data_ptr(), 4, 7)              # flags already there: returns at once
    gpu_ctx.synchronize()
    blk = _block(gpu_ctx)
    blk.forward(gpu_ctx, _x(gpu_ctx, 6, 12), 6, False, 1)   # kernels still run
    gpu_ctx.synchronize()


def test_host_feeder_round_trip(gpu_ctx):
    """Pinned host -> device staging and device -> host fetch deliver the bytes they were given."""
    import torch
    from soklyn_b200.pipeline import HostFeeder
    feeder = HostFeeder(gpu_ctx, [(8, 16)], sk.Precision.FP16)
    host = [torch.arange(128, dtype=torch.float16).reshape(8, 16).pin_memory() * (i + 1) for i in range(3)]
    out = torch.empty((8, 16), dtype=torch.float16).pin_memory()
    feeder.stage(1, [host[0]])
    for s in range(1, 4):
        slot = s % 2
        (x,) = feeder.acquire(slot)
        if s < 3:
            feeder.stage(1 - slot, [host[s]])
        feeder.fetch(x, out, 8)
        feeder.release(slot)
        feeder.wait_output()
        assert torch.equal(out, host[s - 1])
    assert feeder.bytes_h2d == 3 * 256 and feeder.bytes_d2h == 3 * 256


@pytest.mark.parametrize("regu,nesterov", [("l1", False), ("l2", True)])
def test_regularisation_and_nesterov_momentum_match_oracle(gpu_ctx, regu, nesterov):
    """L1 / L2 regularisation (applied to the weights without the learning rate, src/cuda/kernel/ffn/
    backward.cu:120-125) and SGD with (Nesterov) momentum over three steps, f32, against the oracle."""
    from oracle import oracle as ok
    rng = np.random.default_rng(21)
    k, n, m = 20, 12, 10
    w = (rng.standard_normal((k, n)) * 0.3).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    t = rng.standard_normal((m, n)).astype(np.float32)
    coeff = 1e-3
    reg = sk.Regularisation.l1(coeff) if regu == "l1" else sk.Regularisation.l2(coeff)
    cfg = sk.LayerInitConfig(sk.Normalisation.LayerNorm, sk.Activation.Identity, reg, 0.0)
    blk = sk.DenseBlock(gpu_ctx, True, k, n, m, _GivenWeights(w), cfg)
    oblk = ok.OracleBlock(w, m, norm="layer", act="identity", regu=regu, regu_coeff=coeff)
    xd, td = sk.Tensor.from_cpu_vector(gpu_ctx, x, x.shape), sk.Tensor.from_cpu_vector(gpu_ctx, t, t.shape)
    opt = sk.Optimiser.SGD(0.9, nesterov)
    for step in range(1, 4):
        blk.forward(gpu_ctx, xd, m, False, step)
        blk.compute_loss(gpu_ctx, td, sk.LossConfig(sk.LossFunc.MeanSquareLoss, sk.Activation.Tanh))
        blk.backward_output(gpu_ctx, xd, sk.TrainContext(opt, opt, m, 0.05, 0.5), step)     # clamp 0.5 on the update
        oblk.forward(x, m, False, step)
        oblk.compute_loss(t, "mse", "tanh")
        oblk.backward_output(x, ok.TrainContext(ok.sgd(0.9, nesterov), ok.sgd(0.9, nesterov), m, 0.05, 0.5), step)
    for name, got in (("w", blk.get_weights()), ("b", blk.get_biases()), ("dv_w", blk.get_dv_weights()),
                      ("norm_w", blk.get_norm_weights()), ("norm_b", blk.get_norm_biases())):
        e = H.relerr(got.download(gpu_ctx).reshape(-1), getattr(oblk, name).reshape(-1))
        assert e <= 2e-5, f"{name}: {e:.2e}"


def test_convert_f16_and_back(gpu_ctx):
    """DenseBlock::convert_f16 / convert_f32 (src/mlp.rs:835-888): the f32 parameters become the masters
    bit for bit, the 16-bit copies are their roundings, moments and gradient tensors move over, training
    continues within the 16-bit tolerance of an f32 network that was never converted, and converting
    back returns the masters."""
    from soklyn_b200.core import Tensor
    from soklyn_b200.ffn import FeedForwardNetwork
    from soklyn_b200.function import Precision
    spec = configs.scaled(configs.CONFIGS[2], dims=(96, 64, 32, 96), batch=48, precision="f32", name="convert")
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    ref_net, _ = H.run_device(gpu_ctx, spec, w, x, t, 3)          # three f32 steps, never converted
    net, _ = H.run_device(gpu_ctx, spec, w, x, t, 2)              # two f32 steps, then convert
    before = [{k: getattr(l, g)().download(gpu_ctx) for k, g in
               (("w", "get_weights"), ("b", "get_biases"), ("dm", "get_dm_weights"), ("out", "get_outputs"))}
              for l in net.get_layers()]
    moments = [l.get_dm_weights() for l in net.get_layers()]
    half = [l.convert_f16(gpu_ctx) for l in net.get_layers()]
    for blk, old, dm in zip(half, before, moments):
        assert blk.precision == Precision.FP16 and blk.get_dm_weights() is dm
        assert np.array_equal(blk.get_master_weights().download(gpu_ctx), old["w"])
        assert np.array_equal(blk.get_master_biases().download(gpu_ctx), old["b"])
        assert np.array_equal(blk.get_weights().download(gpu_ctx), old["w"].astype(np.float16))
        assert np.array_equal(blk.get_outputs().download(gpu_ctx), old["out"].astype(np.float16))
        assert np.array_equal(blk.get_masks().download(gpu_ctx), np.ones_like(old["out"], np.float16))
        with pytest.raises(log.UnsupportedTypeCast):
            blk.convert_f16(gpu_ctx)
    hnet = FeedForwardNetwork(half, spec.dims[0])
    xd = Tensor.from_cpu_vector(gpu_ctx, x, x.shape, Precision.FP16)
    td = Tensor.from_cpu_vector(gpu_ctx, t, t.shape, Precision.FP16)
    outs = hnet.forward(gpu_ctx, xd, spec.batch, False, 3)
    hnet.backward(gpu_ctx, outs, td, xd, spec.loss_config(), spec.train_context(), 3)
    gpu_ctx.synchronize()
    for blk, ref in zip(half, ref_net.get_layers()):
        assert H.relerr(blk.get_outputs().download(gpu_ctx), ref.get_outputs().download(gpu_ctx)) <= 1e-2
        diff = np.abs(blk.get_master_weights().download(gpu_ctx) - ref.get_weights().download(gpu_ctx))
        assert diff.max() <= 2.5 * spec.lr and (diff > 0.1 * spec.lr).mean() <= 0.01
    masters = [l.get_master_weights().download(gpu_ctx) for l in half]
    back = [l.convert_f32(gpu_ctx) for l in half]
    for blk, m in zip(back, masters):
        assert blk.precision == Precision.FP32 and blk.get_master_weights() is None
        assert np.array_equal(blk.get_weights().download(gpu_ctx), m)
        with pytest.raises(log.UnsupportedTypeCast):
            blk.convert_f32(gpu_ctx)
    fnet = FeedForwardNetwork(back, spec.dims[0])
    xf = Tensor.from_cpu_vector(gpu_ctx, x, x.shape)
    assert np.isfinite(fnet.forward(gpu_ctx, xf, spec.batch, False, 4)[-1].download(gpu_ctx)).all()
