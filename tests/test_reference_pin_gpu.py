"""Pin the CPU oracle to the reference: run the reference's OWN kernels (oracle/_ref) on the
GPU and require the oracle to agree with them. Skipped when oracle/_ref was not built."""
import numpy as np
import pytest

import harness as H
from oracle import ref_kernels
from soklyn_b200 import configs
from soklyn_b200.configs import CONFIGS, scaled

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not ref_kernels.available():
        pytest.skip("reference kernels not built (oracle/_ref)")
    ctx = ref_kernels.RefContext(16, 0, sync_each_launch=True)
    yield ctx
    ctx.close()


SPECS = [CONFIGS[1], scaled(CONFIGS[3], dims=(384, 256, 128, 10), batch=96, precision="f32", name="classifier_small_f32"),
         scaled(CONFIGS[4], dims=(256, 512, 256, 512, 256), batch=192, precision="f32", name="wide_ffn_small_f32")]


@pytest.mark.parametrize("spec", SPECS, ids=lambda s: s.name)
def test_oracle_matches_reference_kernels(ref_ctx, spec):
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    onet, oloss = H.run_oracle(spec, w, x, t, 2)
    rnet, rloss = H.run_device(ref_ctx, spec, w, x, t, 2)
    H.compare_states(ref_ctx, spec, rnet, onet, 2e-5, skip=("mask",), steps=2)
    np.testing.assert_allclose(rloss, oloss, rtol=1e-5)
    for rl, ol in zip(rnet.get_layers(), onet.layers):
        assert np.array_equal(rl.get_masks().download(ref_ctx)[: spec.batch], ol.mask[: spec.batch])


def test_product_matches_reference_kernels_f16(ref_ctx, gpu_ctx):
    """The 16-bit product path against the reference's FP32 kernels (the bar north_star sets: 1e-2)."""
    spec16 = scaled(CONFIGS[4], dims=(256, 512, 256, 512, 256), batch=192, name="wide_ffn_small")
    spec32 = scaled(spec16, precision="f32")
    w = configs.make_weights(spec16)
    x, t, _ = configs.make_data(spec16)
    rnet, _ = H.run_device(ref_ctx, spec32, w, x, t, 1)
    dnet, _ = H.run_device(gpu_ctx, spec16, w, x, t, 1)
    for i, (rl, dl) in enumerate(zip(rnet.get_layers(), dnet.get_layers())):
        rs, ds = H.device_state(ref_ctx, rl), H.device_state(gpu_ctx, dl)
        for name in ("out", "grad", "d_prenorm", "dm_w", "dm_b"):
            e = H.relerr(ds[name][: spec16.batch] if name[0] != "d" or name == "d_prenorm" else ds[name],
                         rs[name][: spec16.batch] if name[0] != "d" or name == "d_prenorm" else rs[name])
            assert e <= 1e-2, f"layer {i} {name}: {e:.3e}"
