"""Parity of the CUDA path (through the C ABI) with the CPU oracle, and of the oracle with
the reference's own kernels. Tolerances: f32 tensors within 1e-5 norm-wise relative error;
16-bit path within 1e-2 of the f32 results; dropout masks and argmax bit-exact."""
import numpy as np
import pytest

import harness as H
from oracle import oracle as ok
from soklyn_b200 import configs
from soklyn_b200.configs import CONFIGS, scaled

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
F16_TOL = 1e-2

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


@pytest.mark.parametrize("spec", [CONFIGS[2], SMALL3, SMALL4], ids=lambda s: s.name)
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
    np.testing.assert_allclose(dloss, oloss, rtol=2e-2)
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
