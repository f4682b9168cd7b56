"""Parity of the CUDA path (through the C ABI) with the CPU oracle, and of the oracle with
the reference's own kernels. Tolerances: f32 tensors within 1e-5 norm-wise relative error;
16-bit path within 1e-2 of the f32 results; dropout masks and argmax bit-exact."""
import numpy as np
import pytest

import harness as H
import soklyn_b200 as sk
from oracle import oracle as ok
from soklyn_b200 import configs
from soklyn_b200.configs import CONFIGS, scaled

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
F16_TOL = 1e-2
# 100-step loss curves of the 16-bit path against the f32 oracle. The two are separate training runs whose
# parameters drift apart by the Adam rule of harness.compare_states, and the drift compounds as training
# proceeds: every step's loss within 2e-2 while the oracle's loss is above a tenth of its first value, within
# 1e-1 once it has fallen below (there the absolute difference is a few 1e-3 of the first loss).
CURVE_TOL_16BIT = 2e-2
CURVE_TOL_16BIT_LATE = 1e-1


def assert_curves_agree(dloss, oloss, label):
    d, o = np.array(dloss), np.array(oloss)
    dev = np.abs(d - o) / o
    early = o >= 0.1 * o[0]
    print(f"{label} loss curve: first {d[0]:.4f}/{o[0]:.4f}, last {d[-1]:.4f}/{o[-1]:.4f}, largest relative deviation "
          f"{dev[early].max():.3e} while above a tenth of the first loss, {dev.max():.3e} overall (step {int(dev.argmax()) + 1})")
    assert dev[early].max() <= CURVE_TOL_16BIT, f"{label}: {dev[early].max():.3e} at step {int(np.where(early, dev, 0).argmax()) + 1}"
    assert dev.max() <= CURVE_TOL_16BIT_LATE, f"{label}: {dev.max():.3e} at step {int(dev.argmax()) + 1}"

# reduced-size variants of the BASELINE configs that the CPU oracle finishes in seconds
SMALL3 = scaled(CONFIGS[3], dims=(384, 256, 128, 10), batch=96, name="classifier_small")
SMALL4 = scaled(CONFIGS[4], dims=(256, 512, 256, 512, 256), batch=192, name="wide_ffn_small")
ODD = configs.NetSpec(9, "odd_shapes", (37, 50, 21, 7), ("batch", "rms", "disabled"), ("tanh", "leaky:0.1", "identity"),
                      (0.0, 0.3, 0.0), "f32", "mse", "sigmoid", "adam", 1e-3, 19, "he_normal", "normal", "normal", True)


def f32_variant(spec):
    return scaled(spec, precision="f32")


@pytest.mark.parametrize("spec", [CONFIGS[1], f32_variant(CONFIGS[2]), f32_variant(SMALL3), f32_variant(SMALL4), ODD],
                         ids=lambda s: s.name)
def test_f32_step_matches_oracle(gpu_ctx, spec):
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    for steps in (1, 3):
        onet, oloss = H.run_oracle(spec, w, x, t, steps)
        dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, steps)
        # after the first Adam step the parameters differ within the rule of compare_states,
        # which the following steps carry into every tensor
        tol = F32_TOL if steps == 1 else (5e-5 if spec.optimiser == "sgd" else 5e-4)
        H.compare_states(gpu_ctx, spec, dnet, onet, tol, skip=("mask",), steps=steps)
        np.testing.assert_allclose(dloss, oloss, rtol=tol)
        for dl, ol in zip(dnet.get_layers(), onet.layers):  # dropout masks: bit-exact
            m = dl.get_masks().download(gpu_ctx)[: spec.batch]
            assert np.array_equal(m, ol.mask[: spec.batch])


# batches above the row count from which the dX epilogue hands its column sums to the weight update,
# not a multiple of the 32-row groups those sums are kept in
TALL3 = scaled(CONFIGS[3], dims=(192, 256, 128, 10), batch=1100, name="classifier_tall")
TALL4 = scaled(CONFIGS[4], dims=(128, 256, 128, 256, 128), batch=1100, name="wide_ffn_tall")


@pytest.mark.parametrize("spec", [CONFIGS[2], SMALL3, SMALL4, TALL3, TALL4], ids=lambda s: s.name)
def test_f16_step_within_1e2_of_f32_oracle(gpu_ctx, spec):
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    onet, oloss = H.run_oracle(spec, w, x, t, 1)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 1)
    # moments of Adam after one step are (1-b)*g and (1-b)*g^2: g^2 doubles the relative error
    H.compare_states(gpu_ctx, spec, dnet, onet, F16_TOL, skip=("mask", "dv_w", "dv_b", "dv_nw", "dv_nb"))
    np.testing.assert_allclose(dloss, oloss, rtol=1e-2)
    for dl, ol in zip(dnet.get_layers(), onet.layers):
        m = dl.get_masks().download(gpu_ctx)[: spec.batch].astype(np.float32)
        assert np.array_equal(m != 0, ol.mask[: spec.batch] != 0)


# The regime every benchmark number comes from: each tensor-core GEMM of these networks has 256 to 512
# output tiles, so every one of the 148 persistent CTAs walks several tiles (second TMEM accumulator,
# stage ring carried across tiles, prefetch across chunks, more than one group of tile columns), and
# the batch is above the row count from which the dX epilogue hands its column sums over.
MULTI_TILE_SPECS = [
    scaled(CONFIGS[4], dims=(4096, 4096, 4096), batch=4096, name="multi_tile_rms_silu_f16"),
    scaled(CONFIGS[3], dims=(2048, 4096, 4096, 16), batch=4096, name="multi_tile_layernorm_mish_dropout_f16"),
    scaled(CONFIGS[4], dims=(2048, 4096, 2048), batch=4096, precision="bf16", name="multi_tile_rms_silu_bf16"),
    scaled(CONFIGS[4], dims=(1000, 4040, 3000), batch=3990, name="multi_tile_ragged_f16"),
]


@pytest.mark.parametrize("spec", MULTI_TILE_SPECS, ids=lambda s: s.name)
def test_multi_tile_per_cta_step_matches_oracle(gpu_ctx, spec):
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    onet, oloss = H.run_oracle(spec, w, x, t, 1)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 1)
    tol = F16_TOL if spec.precision == "f16" else 4e-2   # bf16 keeps 8 bits of mantissa
    H.compare_states(gpu_ctx, spec, dnet, onet, tol, skip=("mask", "dv_w", "dv_b", "dv_nw", "dv_nb"))
    np.testing.assert_allclose(dloss, oloss, rtol=tol)
    for dl, ol in zip(dnet.get_layers(), onet.layers):
        m = dl.get_masks().download(gpu_ctx)[: spec.batch].astype(np.float32)
        assert np.array_equal(m != 0, ol.mask[: spec.batch] != 0)


def test_config3_full_size_step_matches_oracle(gpu_ctx):
    """BASELINE config 3 as specified (3072 -> 1024 -> 512 -> 10, batch 512): one whole step."""
    spec = CONFIGS[3]
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    onet, oloss = H.run_oracle(spec, w, x, t, 1)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 1)
    H.compare_states(gpu_ctx, spec, dnet, onet, F16_TOL, skip=("mask", "dv_w", "dv_b", "dv_nw", "dv_nb"))
    np.testing.assert_allclose(dloss, oloss, rtol=F16_TOL)
    for dl, ol in zip(dnet.get_layers(), onet.layers):
        m = dl.get_masks().download(gpu_ctx)[: spec.batch].astype(np.float32)
        assert np.array_equal(m != 0, ol.mask[: spec.batch] != 0)


BCE_F32 = configs.NetSpec(7, "bce_sigmoid_head_f32", (96, 64, 48), ("layer", "disabled"), ("relu", "identity"), (0.0, 0.0),
                          "f32", "bce", "sigmoid", "adam", 1e-3, 80, "he_normal", "u8", "input")
BCE_F16 = configs.NetSpec(7, "bce_sigmoid_head_f16", (784, 256, 64, 256, 784), ("disabled",) * 4,
                          ("silu", "silu", "silu", "identity"), (0.0,) * 4, "f16", "bce", "sigmoid", "adam", 1e-3, 256,
                          "xavier_normal", "u8", "input")


@pytest.mark.parametrize("spec", [BCE_F32, BCE_F16], ids=lambda s: s.name)
def test_bce_sigmoid_head_matches_oracle(gpu_ctx, spec):
    """Binary cross-entropy on a Sigmoid head (ffn/backward.cu:40-42), the autoencoder example's loss:
    delta = sigmoid(out) - target without the activation derivative."""
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    t = np.ascontiguousarray(t[:, : spec.dims[-1]])   # targets in [0, 1]: the leading columns of the input
    tol = F32_TOL if spec.precision == "f32" else F16_TOL
    onet, oloss = H.run_oracle(spec, w, x, t, 1)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 1)
    skip = ("mask",) if spec.precision == "f32" else ("mask", "dv_w", "dv_b", "dv_nw", "dv_nb")
    H.compare_states(gpu_ctx, spec, dnet, onet, tol, skip=skip)
    np.testing.assert_allclose(dloss, oloss, rtol=tol)
    # the delta itself, element for element: sigmoid(out) - target
    last = dnet.get_layers()[-1]
    out = last.get_outputs().download(gpu_ctx)[: spec.batch].astype(np.float64)
    want = 1.0 / (1.0 + np.exp(-out)) - t
    got = last.get_grads().download(gpu_ctx)[: spec.batch]
    assert H.relerr(got, want) <= (2e-6 if spec.precision == "f32" else 2e-3)


def test_loss_curve_100_steps_f32(gpu_ctx):
    spec = CONFIGS[1]
    w = configs.make_weights(spec)
    x, t, labels = configs.make_data(spec)
    onet, oloss = H.run_oracle(spec, w, x, t, 100)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 100)
    np.testing.assert_allclose(dloss, oloss, rtol=1e-4)
    assert dloss[-1] < 0.7 * dloss[0]
    out = dnet.get_layers()[-1].get_preact_outputs().download(gpu_ctx)[: spec.batch]
    assert np.array_equal(ok.argmax_last(out), ok.argmax_last(onet.layers[-1].preact[: spec.batch]))


def test_loss_curve_100_steps_f16(gpu_ctx):
    spec = CONFIGS[2]
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    onet, oloss = H.run_oracle(spec, w, x, t, 100)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 100)
    assert_curves_agree(dloss, oloss, "config 2")
    assert dloss[-1] < dloss[0]


def test_loss_curve_100_steps_config3(gpu_ctx):
    """Config 3 at full size over its whole cosine schedule (10 warm-up steps, 100 in total), with
    LayerNorm, Mish and dropout: the 16-bit curve against the f32 oracle's."""
    spec = CONFIGS[3]
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    onet, oloss = H.run_oracle(spec, w, x, t, 100)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 100)
    assert_curves_agree(dloss, oloss, "config 3")
    assert dloss[-1] < 0.5 * dloss[0]


def test_loss_curve_100_steps_reduced_config4(gpu_ctx):
    """The wide network's recipe (RMSNorm + SiLU, MSE, Adam) at a size the CPU oracle can step 100 times."""
    spec = scaled(CONFIGS[4], dims=(256, 1024, 256, 1024, 256), batch=384, name="wide_ffn_reduced")
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    onet, oloss = H.run_oracle(spec, w, x, t, 100)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 100)
    assert_curves_agree(dloss, oloss, "reduced config 4")
    assert dloss[-1] < dloss[0]


def test_dropout_mask_bit_exact_full_size(gpu_ctx):
    """Config 3 at its full width: every mask element equals the oracle's hash decision."""
    spec = CONFIGS[3]
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    from soklyn_b200.core import Tensor
    net = H.build_device(gpu_ctx, spec, w)
    xd = Tensor.from_cpu_vector(gpu_ctx, x, x.shape, spec.prec())
    net.forward(gpu_ctx, xd, spec.batch, True, 7)
    L = ok.lib()
    for i, layer in enumerate(net.get_layers()[:2]):
        m = layer.get_masks().download(gpu_ctx).astype(np.float32)
        seed = ok.scramble_seed(7, spec.id_stride() * i)
        rows, cols = np.meshgrid(np.arange(spec.batch, dtype=np.uint32), np.arange(m.shape[1], dtype=np.uint32), indexing="ij")
        s = (rows * np.uint32(1103515245)) ^ (cols * np.uint32(0x4C957F2D)) ^ (np.uint32(seed) + rows * np.uint32(7))
        s ^= s >> np.uint32(17)
        s = s * np.uint32(1103515245) + np.uint32(12345)
        s ^= s >> np.uint32(15)
        keep = (s.astype(np.float32) / np.float32(4294967296.0)) >= np.float32(0.1)
        assert np.array_equal(m != 0, keep)
        assert abs(keep.mean() - 0.9) < 0.01


TC_SPECS = [
    SMALL4,
    scaled(CONFIGS[4], dims=(72, 200, 136, 24), batch=100, name="tc_ragged_tiles"),          # no dimension fills a tile
    scaled(CONFIGS[3], dims=(512, 384, 256, 64), batch=300, name="tc_layernorm_dropout"),
    scaled(CONFIGS[2], dims=(784, 256, 64, 256, 784), batch=256, name="tc_autoencoder"),
    scaled(CONFIGS[4], dims=(256, 1024, 256), batch=640, precision="bf16", name="tc_bf16"),
]


@pytest.mark.parametrize("spec", TC_SPECS, ids=lambda s: s.name)
def test_tensor_core_gemm_matches_ffma_gemm(gpu_ctx, spec):
    """The tcgen05 kernel and the FFMA kernel compute the same products from the same 16-bit
    operands with f32 accumulation; only the summation order differs."""
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    try:
        gpu_ctx.set_gemm_engine(True)
        fnet, floss = H.run_device(gpu_ctx, spec, w, x, t, 2)
        fstate = [H.device_state(gpu_ctx, l) for l in fnet.get_layers()]
    finally:
        gpu_ctx.set_gemm_engine(False)
    tnet, tloss = H.run_device(gpu_ctx, spec, w, x, t, 2)
    tstate = [H.device_state(gpu_ctx, l) for l in tnet.get_layers()]
    np.testing.assert_allclose(tloss, floss, rtol=2e-3)
    for i, (a, b) in enumerate(zip(tstate, fstate)):
        for name in ("prenorm", "preact", "out", "grad", "d_prenorm", "dm_w", "dm_b", "d_norm_w"):
            if name in a:
                e = H.relerr(a[name], b[name])
                tol = 4e-3 if spec.precision == "f16" else 1.6e-2   # a couple of ulps of the storage type
                assert e <= tol, f"layer {i} {name}: tensor-core vs FFMA relative error {e:.3e}"
        assert np.array_equal(a["mask"], b["mask"])


def test_two_heads_on_one_trunk_match_oracle(gpu_ctx):
    """The reference's multi-head pattern (examples/cifar_ten_train.rs:175-244): two output blocks read the
    same trunk output, each step trains one of them and back-propagates it into the trunk through the
    per-block calls, the second head with its own learning rate and a gradient clamp."""
    import soklyn_b200 as sk
    from soklyn_b200.core import Tensor, reset_tensor_ids
    from soklyn_b200.context import LayerInitConfig, LossConfig, TrainContext
    from soklyn_b200.function import Activation, LossFunc, Normalisation, Optimiser, Regularisation
    batch, dims, heads = 40, (72, 64, 48), (10, 2)
    rng = np.random.Generator(np.random.PCG64(77))
    ws = [rng.standard_normal((dims[i], dims[i + 1]), dtype=np.float32) * np.float32(np.sqrt(2.0 / dims[i])) for i in range(2)]
    ws += [rng.standard_normal((dims[2], h), dtype=np.float32) * np.float32(np.sqrt(2.0 / dims[2])) for h in heads]
    x = rng.standard_normal((batch, dims[0]), dtype=np.float32)
    labels = [rng.integers(0, h, batch) for h in heads]
    targets = [np.eye(h, dtype=np.float32)[l] for h, l in zip(heads, labels)]

    reset_tensor_ids(0)
    cfgs = [LayerInitConfig(Normalisation.LayerNorm, Activation.Mish, Regularisation.none(), 0.2)] * 2 + [LayerInitConfig()] * 2
    shapes = [(dims[0], dims[1]), (dims[1], dims[2]), (dims[2], heads[0]), (dims[2], heads[1])]
    dev = [sk.DenseBlock(gpu_ctx, True, k, n, batch, configs._GivenWeights(w), c) for (k, n), w, c in zip(shapes, ws, cfgs)]
    ora = [ok.OracleBlock(w, batch, norm="layer" if i < 2 else "disabled", act="mish" if i < 2 else "identity",
                          mask_coeff=0.2 if i < 2 else 0.0, tensor_id=dev[i].get_weights().get_id()) for i, w in enumerate(ws)]
    xd = Tensor.from_cpu_vector(gpu_ctx, x, x.shape)
    td = [Tensor.from_cpu_vector(gpu_ctx, t, t.shape) for t in targets]
    loss = LossConfig(LossFunc.CrossEntropyLoss, Activation.Softmax)
    for step in range(1, 5):
        head = 0 if step % 2 else 1
        lr, clamp = (1e-3, 0.05) if head == 0 else (1e-5, 1e-6)
        # device: forward through the trunk and both heads, then the chosen head backwards
        o0 = dev[0].forward(gpu_ctx, xd, batch, True, step)
        o1 = dev[1].forward(gpu_ctx, o0, batch, True, step)
        for h in (2, 3):
            dev[h].forward(gpu_ctx, o1, batch, True, step)
        tc = TrainContext(Optimiser.Adam(), Optimiser.Adam(), batch, lr, clamp)
        dev[2 + head].compute_loss(gpu_ctx, td[head], loss)
        dev[2 + head].backward_output(gpu_ctx, o1, tc, step)
        dev[1].backward_hidden(gpu_ctx, dev[2 + head], o0, tc, step)
        dev[0].backward_hidden(gpu_ctx, dev[1], xd, tc, step)
        # oracle: the same calls
        p0 = ora[0].forward(x, batch, True, step)
        p1 = ora[1].forward(p0, batch, True, step)
        for h in (2, 3):
            ora[h].forward(p1, batch, True, step)
        oc = ok.TrainContext(ok.adam(), ok.adam(), batch, lr, clamp)
        ora[2 + head].compute_loss(targets[head], "ce", "softmax")
        ora[2 + head].backward_output(p1, oc, step)
        ora[1].backward_hidden(ora[2 + head], p0, oc, step)
        ora[0].backward_hidden(ora[1], x, oc, step)
    gpu_ctx.synchronize()
    for i, (d, o) in enumerate(zip(dev, ora)):
        got, ref = H.device_state(gpu_ctx, d), o.state()
        assert np.array_equal(got["mask"], ref["mask"]), f"block {i} mask"
        for name in ("out", "preact", "grad", "d_prenorm", "dm_w", "dm_nw"):
            assert H.relerr(got[name].reshape(ref[name].shape), ref[name]) <= 5e-4, f"block {i} {name}"
        for name in ("w", "b", "norm_w", "norm_b"):   # Adam: distance from the oracle in units of the largest rate
            assert np.abs(got[name].reshape(ref[name].shape) - ref[name]).max() <= 0.1 * 1e-3 * 4, f"block {i} {name}"


@pytest.mark.parametrize("spec", [TALL4, TALL3], ids=lambda s: s.name)
def test_lean_backward_gives_bit_identical_parameters(gpu_ctx, spec):
    """SK_OPTION_LEAN_BACKWARD skips the stores of grad, the f32 d_prenorm, d_norm_w and d_norm_b in hidden
    blocks whose column sums are taken in the dX epilogue. Nothing in the backward pass reads them, so three
    training steps must leave every parameter, master copy and moment bit for bit as the default run does."""
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    dnet, dloss = H.run_device(gpu_ctx, spec, w, x, t, 3)
    want = [H.device_state(gpu_ctx, l) for l in dnet.get_layers()]
    try:
        gpu_ctx.set_lean_backward(True)
        lnet, lloss = H.run_device(gpu_ctx, spec, w, x, t, 3)
        got = [H.device_state(gpu_ctx, l) for l in lnet.get_layers()]
    finally:
        gpu_ctx.set_lean_backward(False)
    assert lloss == dloss
    names = ("w", "b", "norm_w", "norm_b", "dv_w", "dm_w", "dv_b", "dm_b", "dv_nw", "dm_nw", "dv_nb", "dm_nb", "out", "mask")
    for i, (a, b) in enumerate(zip(got, want)):
        for name in names:
            if name in a:
                assert np.array_equal(a[name], b[name]), f"layer {i} {name} differs between the lean and the default run"
    # and the skipped tensors really were skipped in the hidden blocks (they keep their initial zeros)
    assert not np.any(got[0]["grad"]) and np.any(want[0]["grad"])


def test_f32_tensor_core_option_stays_within_5e5_of_the_ffma_path(gpu_ctx):
    """SK_OPTION_F32_TENSOR_CORES: large f32 products through three bf16 parts per operand and six partial
    products on the tensor cores, summed over K in registers with round-to-nearest adds (the tensor pipe
    truncates when it adds into its f32 accumulator, so the accumulators are closed every eight 64-deep K steps).
    Single products land within 3e-6 of the f32 oracle; through a LayerNorm backward that amplifies the
    difference up to 1.5e-5, above the 1e-5 of the default FFMA path, so the option is off by default. What it
    must meet: 5e-5 on every tensor, bit-equal dropout masks and a loss within 1e-5."""
    spec = scaled(CONFIGS[3], dims=(1024, 1024, 512, 16), batch=1024, precision="f32", name="f32_tensor_core_option")
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    before = gpu_ctx.launch_count()
    fnet, floss = H.run_device(gpu_ctx, spec, w, x, t, 1)
    plain_launches = gpu_ctx.launch_count() - before
    want = [H.device_state(gpu_ctx, l) for l in fnet.get_layers()]
    try:
        gpu_ctx.set_f32_tensor_cores(True)
        before = gpu_ctx.launch_count()
        tnet, tloss = H.run_device(gpu_ctx, spec, w, x, t, 1)
        launches = gpu_ctx.launch_count() - before
        got = [H.device_state(gpu_ctx, l) for l in tnet.get_layers()]
    finally:
        gpu_ctx.set_f32_tensor_cores(False)
    np.testing.assert_allclose(tloss, floss, rtol=1e-5)
    worst = 0.0
    for i, (a, b) in enumerate(zip(got, want)):
        assert np.array_equal(a["mask"], b["mask"])
        for name in ("prenorm", "preact", "out", "grad", "d_prenorm", "dm_w", "dm_b", "d_norm_w"):
            if name in a:
                e = H.relerr(a[name], b[name])
                worst = max(worst, e)
                assert e <= 5e-5, f"layer {i} {name}: {e:.3e}"
    assert worst > 0.0, "the tensor-core path did not run (results are bit-identical to the FFMA path)"
    assert launches >= plain_launches + 8      # the split kernels ran: two more launches per large product


@pytest.mark.parametrize("k", [4096, 16384])
def test_f32_tensor_core_option_has_no_truncation_bias_on_long_positive_sums(gpu_ctx, k):
    """All-positive operands are the worst case for an accumulator that truncates: summed in TMEM alone the
    error grew linearly with K (2.6e-5 of the result at K = 4096, 1.1e-4 at 16384). With the sum over K kept in
    registers every element stays within 2e-6 of the float64 product at both depths."""
    from soklyn_b200.configs import _GivenWeights
    from soklyn_b200.core import Tensor
    m = n = 512
    rng = np.random.default_rng(5)
    wt = rng.random((k, n), dtype=np.float32)
    xv = rng.random((m, k), dtype=np.float32)
    ref = xv.astype(np.float64) @ wt.astype(np.float64)
    ref = ref / (1.0 + np.exp(-ref))              # SiLU; the products are in the hundreds, where it is the identity to 1e-40
    cfg = sk.LayerInitConfig(sk.Normalisation.Disabled, sk.Activation.SiLU, sk.Regularisation.none(), 0.0)
    try:
        gpu_ctx.set_f32_tensor_cores(True)
        gpu_ctx.reserve(6 * (m + n) * k * 2 + 4096)   # the three bf16 parts of both operands live in the workspace
        blk = sk.DenseBlock(gpu_ctx, True, k, n, m, _GivenWeights(wt), cfg, sk.Precision.FP32)
        xx = Tensor.from_cpu_vector(gpu_ctx, xv, (m, k), sk.Precision.FP32)
        before = gpu_ctx.launch_count()
        blk.forward(gpu_ctx, xx, m, False, 1)
        assert gpu_ctx.launch_count() - before >= 3   # two split kernels and the product
        got = H.device_state(gpu_ctx, blk)["out"].reshape(-1, n)[:m].astype(np.float64)
    finally:
        gpu_ctx.set_f32_tensor_cores(False)
    rel = np.abs(got - ref) / np.abs(ref)
    assert rel.max() <= 2e-6, f"K={k}: max relative error {rel.max():.2e}"
