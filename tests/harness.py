"""Shared test machinery: build the same seeded network on the CPU oracle and on a
device context (product library or reference kernels), run training steps, compare."""
from __future__ import annotations

import numpy as np

from oracle import oracle as ok
from soklyn_b200 import configs
from soklyn_b200.core import Tensor, reset_tensor_ids
from soklyn_b200.scheduler import CosineDecayLR

STATE_DEVICE = {  # oracle name -> DenseBlock getter
    "w": "get_weights", "b": "get_biases", "dv_w": "get_dv_weights", "dm_w": "get_dm_weights",
    "dv_b": "get_dv_biases", "dm_b": "get_dm_biases", "norm_w": "get_norm_weights", "norm_b": "get_norm_biases",
    "dv_nw": "get_dv_norm_weights", "dm_nw": "get_dm_norm_weights", "dv_nb": "get_dv_norm_biases",
    "dm_nb": "get_dm_norm_biases", "out": "get_outputs", "predrop": "get_predrop_outputs",
    "preact": "get_preact_outputs", "centered": "get_centered_outputs", "prenorm": "get_prenorm_outputs",
    "rstd": "get_norm_rstd", "grad": "get_grads", "d_prenorm": "get_delta_prenorm_out",
    "d_norm_w": "get_norm_weights_grad", "d_norm_b": "get_norm_biases_grad", "mask": "get_masks",
}


def relerr(a: np.ndarray, b: np.ndarray) -> float:
    """Norm-wise relative error max|a-b| / max|b| (element-wise relative error explodes near zero)."""
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    denom = max(float(np.abs(b).max()), 1e-30)
    return float(np.abs(a - b).max() / denom)


def _oracle_act(spec, i):
    a = spec.acts[i]
    return ("leaky_relu", float(a.split(":")[1])) if a.startswith("leaky") else (a, 0.0)


def build_oracle(spec, weights, max_batch=None):
    mb = spec.batch if max_batch is None else max_batch
    layers = []
    for i in range(spec.layers):
        act, leaky = _oracle_act(spec, i)
        layers.append(ok.OracleBlock(weights[i], mb, norm=spec.norms[i], act=act, leaky=leaky,
                                     mask_coeff=spec.mask_coeffs[i], tensor_id=spec.id_stride() * i))
    return ok.OracleFFN(layers)


def build_device(ctx, spec, weights, max_batch=None):
    """Network on a device context, with the tensor ids a fresh reference process would give."""
    reset_tensor_ids(0)
    net = configs.build_network(ctx, spec, weights, max_batch)
    for i, layer in enumerate(net.get_layers()):
        assert layer.get_weights().get_id() == spec.id_stride() * i
    return net


def _oracle_optim(spec):
    o = ok.sgd(0.0, False) if spec.optimiser == "sgd" else ok.adam(0.9, 0.999, 1e-8)
    return [o] * spec.layers


def lr_schedule(spec, steps):
    if spec.cosine is None:
        return [spec.lr] * steps
    s = CosineDecayLR(*spec.cosine)
    return [s.step() for _ in range(steps)]


def run_oracle(spec, weights, x, t, steps, max_batch=None):
    net = build_oracle(spec, weights, max_batch)
    losses, opt = [], _oracle_optim(spec)
    lrs = lr_schedule(spec, steps)
    for s in range(1, steps + 1):
        outs = net.forward(x, spec.batch, spec.use_dropout, s)
        losses.append(configs.host_loss(spec, outs[-1][: spec.batch].copy(), t[: spec.batch]))
        net.backward(outs, t, x, spec.loss, spec.loss_act, opt, opt, spec.batch, lrs[s - 1], s)
    return net, losses


def run_device(ctx, spec, weights, x, t, steps, max_batch=None):
    net = build_device(ctx, spec, weights, max_batch)
    prec = spec.prec()
    xd = Tensor.from_cpu_vector(ctx, x, x.shape, prec)
    td = Tensor.from_cpu_vector(ctx, t, t.shape, prec)
    losses = []
    lrs = lr_schedule(spec, steps)
    for s in range(1, steps + 1):
        outs = net.forward(ctx, xd, spec.batch, spec.use_dropout, s)
        out_host = outs[-1].download(ctx)[: spec.batch].astype(np.float32)
        losses.append(configs.host_loss(spec, out_host, t[: spec.batch]))
        net.backward(ctx, outs, td, xd, spec.loss_config(), spec.train_context(lr=lrs[s - 1]), s)
    ctx.synchronize()
    return net, losses


def device_state(ctx, layer) -> dict:
    out = {}
    for name, getter in STATE_DEVICE.items():
        t = getattr(layer, getter)()
        if t is not None:
            out[name] = t.download(ctx).astype(np.float32)
    if layer.get_master_weights() is not None:  # 16-bit: compare the f32 masters as the parameters
        out["w"] = layer.get_master_weights().download(ctx)
        out["b"] = layer.get_master_biases().download(ctx)
        out["norm_w"] = layer.get_master_norm_weights().download(ctx)
        out["norm_b"] = layer.get_master_norm_biases().download(ctx)
    return out


PARAMS = ("w", "b", "norm_w", "norm_b")


def compare_states(ctx, spec, dev_net, oracle_net, tol, skip=(), steps=1):
    """Max norm-wise relative error per tensor name over all layers; asserts each <= tol. Parameters updated
    by Adam are reported under "adam_moved_lr:<name>" as their largest distance from the oracle in units of
    the learning rate, not as a relative error.

    Parameters updated by Adam get their own rule. Adam's step is lr*m/(sqrt(v)+eps); at
    step 1 that is lr*g/(|g|+eps), about lr*sign(g): an element whose gradient lies within
    rounding noise of zero can land anywhere in [-lr, +lr] whichever (correct) summation
    order produced it, and the reference's own GPU kernels differ from a CPU run in the same
    way. So for Adam the gradient is checked through the first moment dm = (1-b1)*g at `tol`,
    and the parameters by how far they moved in units of lr: in f32 every element within
    0.1*lr per step; in 16-bit 99% of the elements within 0.1*lr and all within 2.5*lr per step.
    """
    worst = {}
    lr_max = max(lr_schedule(spec, max(steps, 1)))
    for i, (dl, ol) in enumerate(zip(dev_net.get_layers(), oracle_net.layers)):
        ds, os_ = device_state(ctx, dl), ol.state()
        rows = spec.batch
        for name, ref in os_.items():
            if name in skip or name not in ds:
                continue
            got = ds[name].reshape(ref.shape) if ds[name].size == ref.size else ds[name]
            if ref.ndim == 2 and ref.shape[0] == ol.max_batch and name != "w":
                got, ref = got[:rows], ref[:rows]
            if name == "rstd":
                n = rows if spec.norms[i] in ("rms", "layer") else (ol.N if spec.norms[i] == "batch" else 0)
                got, ref = got.reshape(-1)[:n], ref[:n]
                if n == 0:
                    continue
            e = relerr(got, ref)
            if name in PARAMS and spec.optimiser == "adam":
                # reported apart from the tensor errors: distance from the oracle in units of the learning rate
                moved = float((np.abs(got.astype(np.float64) - ref.astype(np.float64)) / lr_max).max())
                worst["adam_moved_lr:" + name] = max(worst.get("adam_moved_lr:" + name, 0.0), moved)
            else:
                worst[name] = max(worst.get(name, 0.0), e)
            if name in PARAMS and spec.optimiser == "adam" and e > tol:
                diff = np.abs(got.astype(np.float64) - ref.astype(np.float64)) / lr_max
                if tol <= 1e-3:
                    assert diff.max() <= 0.1 * steps, f"layer {i} {name}: moved {diff.max():.3f} lr from the oracle"
                else:
                    assert (diff > 0.1 * steps).mean() <= 0.01 and diff.max() <= 2.5 * steps, \
                        f"layer {i} {name}: {100 * (diff > 0.1 * steps).mean():.2f}% beyond 0.1 lr, max {diff.max():.2f} lr"
                continue
            assert e <= tol, f"layer {i} tensor {name}: relative error {e:.3e} > {tol:.1e}"
    return worst
