"""The C++ host mirror trains the same networks as the Python mirror, bit for bit (both are
thin layers over the same C ABI), and so inherits its parity with the CPU oracle; the
oracle is also compared directly. The driver runs the mirror's error-behaviour checks on the
device before training."""
import numpy as np
import pytest

import cpp_host
import harness as H
from soklyn_b200 import configs
from soklyn_b200.configs import CONFIGS, scaled

pytestmark = pytest.mark.gpu

SMALL3 = scaled(CONFIGS[3], dims=(384, 256, 128, 10), batch=96, name="classifier_small")
SMALL4 = scaled(CONFIGS[4], dims=(256, 512, 256, 512, 256), batch=192, name="wide_ffn_small")
ODD = configs.NetSpec(9, "odd_shapes", (37, 50, 21, 7), ("batch", "rms", "disabled"), ("tanh", "leaky:0.1", "identity"),
                      (0.0, 0.3, 0.0), "f32", "mse", "sigmoid", "adam", 1e-3, 19, "he_normal", "normal", "normal", True)
GETTERS = {"out": "get_outputs", "preact": "get_preact_outputs", "mask": "get_masks", "grad": "get_grads",
           "d_prenorm": "get_delta_prenorm_out", "dm_w": "get_dm_weights", "dv_w": "get_dv_weights"}
MASTERS = {"w": ("get_master_weights", "get_weights"), "b": ("get_master_biases", "get_biases"),
           "norm_w": ("get_master_norm_weights", "get_norm_weights"), "norm_b": ("get_master_norm_biases", "get_norm_biases")}


def _cpp_train(tmp_path, spec, w, x, t, steps, fused):
    # fused: bit 0 = whole-network native calls, bit 1 = every step recorded and launched as one CUDA graph
    src, dst = str(tmp_path / "in.bin"), str(tmp_path / f"out_{int(fused)}.bin")
    cpp_host.write_spec(src, spec, w, x, t, steps, fused=fused)
    r = cpp_host.run("train", src, dst)
    assert r.returncode == 0, r.stdout + r.stderr
    return cpp_host.read_records(dst)


@pytest.mark.parametrize("spec,steps", [(CONFIGS[1], 5), (CONFIGS[2], 3), (SMALL3, 4), (SMALL4, 2), (ODD, 3)],
                         ids=lambda v: getattr(v, "name", str(v)))
def test_cpp_mirror_equals_python_mirror(gpu_ctx, tmp_path, spec, steps):
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    recs = _cpp_train(tmp_path, spec, w, x, t, steps, fused=True)
    unfused = _cpp_train(tmp_path, spec, w, x, t, steps, fused=False)
    # Per-layer calls and whole-network calls run the same kernels, except that the whole-network call
    # takes the column sums of a hidden layer in the dX epilogue (another summation order): parameters may
    # differ by rounding, within the rule the oracle comparison uses.
    assert [n for n, _ in recs] == [n for n, _ in unfused]
    # GpuContext::StepGraph around every step: the same kernels with the same arguments, bit for bit. The
    # per-step output record is left out: inside a recorded step nothing can be read back, so the driver reads
    # it after backward, which has turned the output block's values into softmax / sigmoid of them in place.
    graphed = _cpp_train(tmp_path, spec, w, x, t, steps, fused=3)
    assert [n for n, _ in recs] == [n for n, _ in graphed]
    for (name, a), (_, g) in zip(recs, graphed):
        if name != "step_out":
            assert np.array_equal(a, g, equal_nan=True), f"{name} differs under the step graph"
    lr_max = max(H.lr_schedule(spec, steps))
    for (name, a), (_, b) in zip(recs, unfused):
        kind = name.split(".")[-1]
        if kind in ("id", "mask"):
            assert np.array_equal(a, b), name
        elif kind in ("w", "b", "norm_w", "norm_b"):
            assert np.abs(a - b).max() <= 2.5 * lr_max * steps, name
        elif kind != "dv_w":
            assert H.relerr(a, b) <= (1e-4 if spec.precision == "f32" else 2e-2), name

    # the Python mirror, recording the last layer's output of every step
    net = H.build_device(gpu_ctx, spec, w)
    from soklyn_b200.core import Tensor
    xd = Tensor.from_cpu_vector(gpu_ctx, x, x.shape, spec.prec())
    td = Tensor.from_cpu_vector(gpu_ctx, t, t.shape, spec.prec())
    lrs = H.lr_schedule(spec, steps)
    step_outs = []
    for s in range(1, steps + 1):
        outs = net.forward(gpu_ctx, xd, spec.batch, spec.use_dropout, s)
        step_outs.append(outs[-1].download(gpu_ctx).astype(np.float32).reshape(-1))
        net.backward(gpu_ctx, outs, td, xd, spec.loss_config(), spec.train_context(lr=lrs[s - 1]), s)
    gpu_ctx.synchronize()

    got_steps = [v for n, v in recs if n == "step_out"]
    assert len(got_steps) == steps
    for s, (a, b) in enumerate(zip(got_steps, step_outs)):
        assert np.array_equal(a, b), f"step {s + 1}: last layer output differs from the Python mirror"
    final = dict(recs)
    for i, layer in enumerate(net.get_layers()):
        assert int(final[f"l{i}.id"][0]) == spec.id_stride() * i      # tensor ids as a fresh reference process
        for name, getter in GETTERS.items():
            ref = getattr(layer, getter)().download(gpu_ctx).astype(np.float32).reshape(-1)
            assert np.array_equal(final[f"l{i}.{name}"], ref, equal_nan=True), f"layer {i} {name}"
        for name, (master, plain) in MASTERS.items():
            tns = getattr(layer, master)() or getattr(layer, plain)()
            assert np.array_equal(final[f"l{i}.{name}"], tns.download(gpu_ctx).astype(np.float32).reshape(-1)), f"layer {i} {name}"


def test_cpp_mirror_against_oracle_f32(gpu_ctx, tmp_path):
    """Directly against the CPU oracle: one SGD step of the f32 MLP within 1e-5, dropout mask bit-exact."""
    spec = CONFIGS[1]
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    onet, _ = H.run_oracle(spec, w, x, t, 1)
    final = dict(_cpp_train(tmp_path, spec, w, x, t, 1, fused=True))
    for i, ol in enumerate(onet.layers):
        st = ol.state()
        for name in ("w", "b", "out", "preact", "grad", "d_prenorm"):
            got = final[f"l{i}.{name}"]
            ref = st[name].reshape(-1)[: got.size] if st[name].size >= got.size else st[name].reshape(-1)
            assert H.relerr(got[: ref.size], ref) <= 1e-5, f"layer {i} {name}"
        assert np.array_equal(final[f"l{i}.mask"], st["mask"].reshape(-1))
