"""Generate tests/golden/reference_kernels.npz by running the REFERENCE's own CUDA kernels
(oracle/_ref, see oracle/build_ref.py) on seeded configurations. Needs a GPU:

    python tests/golden/make_golden.py [output.npz]

Inputs and weights are regenerated from seeds by soklyn_b200.configs, so only outputs are
stored: every tensor of every layer after `steps` training steps, sampled with a fixed
stride (at most ~160 values per tensor) plus its f64 sum and absolute sum.
"""
import os
import sys

from dataclasses import replace

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from soklyn_b200 import configs  # noqa: E402
from soklyn_b200.configs import CONFIGS, scaled  # noqa: E402


def golden_specs():
    small3 = scaled(CONFIGS[3], dims=(384, 256, 128, 10), batch=96, precision="f32", name="classifier_small_f32")
    # the committed vectors of this network were taken with Adam at lr 1e-3 (at this size it trains at that rate)
    small4 = replace(scaled(CONFIGS[4], dims=(256, 512, 256, 512, 256), batch=192, precision="f32", name="wide_ffn_small_f32"),
                     lr=1e-3)
    odd = configs.NetSpec(9, "odd_shapes", (37, 50, 21, 7), ("batch", "rms", "disabled"),
                          ("tanh", "leaky:0.1", "identity"), (0.0, 0.3, 0.0), "f32", "mse", "sigmoid", "adam", 1e-3, 19,
                          "he_normal", "normal", "normal", True)
    bce = configs.NetSpec(8, "bce_head", (48, 32, 48), ("layer", "disabled"), ("sigmoid", "identity"), (0.0, 0.0),
                          "f32", "bce", "sigmoid", "sgd", 0.05, 24, "xavier_uniform", "u8", "input")
    return [(CONFIGS[1], 2), (scaled(CONFIGS[2], precision="f32", name="autoencoder_f32"), 2), (small3, 2), (small4, 2),
            (odd, 2), (bce, 2)]


def sample(a: np.ndarray) -> np.ndarray:
    flat = np.asarray(a, np.float32).reshape(-1)
    stride = max(1, flat.size // 160)
    return np.concatenate([flat[::stride], np.array([flat.astype(np.float64).sum(), np.abs(flat.astype(np.float64)).sum()],
                                                    np.float64).astype(np.float32)])


def digest(states: list, spec) -> dict:
    out = {}
    for i, st in enumerate(states):
        for name, arr in st.items():
            a = np.asarray(arr)
            if a.ndim == 2 and a.shape[0] >= spec.batch and name not in ("w", "dv_w", "dm_w"):
                a = a[: spec.batch]
            if name == "rstd":
                n = spec.batch if spec.norms[i] in ("rms", "layer") else (spec.dims[i + 1] if spec.norms[i] == "batch" else 0)
                a = a.reshape(-1)[:n]
            out[f"{spec.name}/L{i}/{name}"] = sample(a) if a.size else np.zeros(0, np.float32)
    return out


def main():
    import harness as H
    from oracle.ref_kernels import RefContext
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_kernels.npz")
    ctx = RefContext(16, 0, sync_each_launch=True)
    blob = {}
    for spec, steps in golden_specs():
        w = configs.make_weights(spec)
        x, t, _ = configs.make_data(spec)
        net, losses = H.run_device(ctx, spec, w, x, t, steps)
        states = [H.device_state(ctx, layer) for layer in net.get_layers()]
        blob.update(digest(states, spec))
        blob[f"{spec.name}/losses"] = np.asarray(losses, np.float32)
        print(spec.name, "losses", losses)
    os.makedirs(os.path.dirname(out_path), exist_ok=True)
    np.savez_compressed(out_path, **blob)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main()
