"""The CPU oracle against (a) the vectors the reference's own kernels produced
(tests/golden/reference_kernels.npz, made by tests/golden/make_golden.py on a GPU),
(b) known answers worked out from the reference's formulas, (c) finite differences."""
import os

import numpy as np
import pytest

import harness as H
from oracle import oracle as ok
from soklyn_b200 import configs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.npz")


def test_hash_known_answers():
    L = ok.lib()
    def ref(col, row, seed):   # src/cuda/kernel/math.cuh:45-53 in Python integers
        m = 0xFFFFFFFF
        s = ((row * 1103515245) ^ (col * 6364136223846793005) ^ seed) & m
        s ^= s >> 17
        s = (s * 1103515245 + 12345) & m
        s ^= s >> 15
        return np.float32(s) / np.float32(0xFFFFFFFF)
    for col, row, seed in [(0, 0, 0), (1, 2, 3), (783, 63, 0xDEADBEEF), (16383, 8191, 12345), (5, 0xFFFFFF, 7)]:
        assert np.float32(L.ok_rand(col, row, seed)) == ref(col, row, seed)
    vals = np.array([L.ok_rand(c, r, 99) for c in range(64) for r in range(64)])
    assert 0.45 < vals.mean() < 0.55 and vals.min() >= 0 and vals.max() <= 1


def test_activation_known_answers():
    L = ok.lib()
    x = 0.7
    sig = 1 / (1 + np.exp(-x))
    assert L.ok_activation(1, x, 0) == pytest.approx(sig, rel=1e-6)
    assert L.ok_activation(2, -x, 0) == 0 and L.ok_activation(2, x, 0) == pytest.approx(x)
    assert L.ok_activation(3, -x, 0.1) == pytest.approx(-0.07, rel=1e-6)
    assert L.ok_activation(4, x, 0) == pytest.approx(np.tanh(x), rel=1e-6)
    assert L.ok_activation(6, x, 0) == pytest.approx(x * sig, rel=1e-6)
    assert L.ok_activation(7, x, 0) == pytest.approx(x * np.tanh(np.log1p(np.exp(x))), rel=1e-5)
    assert L.ok_activation(7, 25.0, 0) == pytest.approx(25.0, rel=1e-6)
    assert L.ok_activation(5, x, 0) == pytest.approx(x) and L.ok_activation(0, x, 0) == pytest.approx(x)


@pytest.mark.parametrize("act", [1, 4, 6, 7])
def test_activation_derivative_is_the_derivative(act):
    L = ok.lib()
    for x in (-1.3, -0.2, 0.4, 2.1):
        h = 1e-3
        num = (L.ok_activation(act, x + h, 0) - L.ok_activation(act, x - h, 0)) / (2 * h)
        got = L.ok_activation_derivative(act, 1.0, L.ok_activation(act, x, 0), x, 0)
        assert got == pytest.approx(num, rel=2e-3, abs=2e-4)


def test_weight_gradient_is_the_mse_gradient():
    """One SGD step without momentum moves W by -lr * dLoss/dW of 0.5*sum((out-t)^2)/M."""
    rng = np.random.default_rng(5)
    m, k, n = 6, 5, 4
    w = rng.standard_normal((k, n)).astype(np.float32) * 0.3
    x = rng.standard_normal((m, k)).astype(np.float32)
    t = rng.standard_normal((m, n)).astype(np.float32)
    blk = ok.OracleBlock(w, m, act="identity")
    net = ok.OracleFFN([blk])
    outs = net.forward(x, m, False, 1)
    net.backward(outs, t, x, "mse", "identity", [ok.sgd()], [ok.sgd()], m, 0.1, 1)
    grad = x.T @ (x @ w - t) / m
    np.testing.assert_allclose(blk.w, w - 0.1 * grad, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(blk.b, -0.1 * (x @ w - t).mean(0), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(blk.d_prenorm, (x @ w - t) * 512, rtol=1e-5, atol=1e-4)


def test_hidden_delta_uses_updated_next_weights():
    rng = np.random.default_rng(6)
    m = 4
    w0 = rng.standard_normal((3, 5)).astype(np.float32)
    w1 = rng.standard_normal((5, 2)).astype(np.float32)
    x = rng.standard_normal((m, 3)).astype(np.float32)
    t = rng.standard_normal((m, 2)).astype(np.float32)
    net = ok.OracleFFN([ok.OracleBlock(w0, m, act="tanh"), ok.OracleBlock(w1, m)])
    outs = net.forward(x, m, False, 1)
    h = outs[0].copy()
    net.backward(outs, t, x, "mse", "identity", [ok.sgd()] * 2, [ok.sgd()] * 2, m, 0.5, 1)
    w1_new = net.layers[1].w
    assert not np.allclose(w1_new, w1)
    delta1 = (h @ w1 - t) * 512
    expect = (delta1 @ w1_new.T) * (1 - h * h)          # ffn.rs:141-163: next layer already stepped
    np.testing.assert_allclose(net.layers[0].grad, expect, rtol=2e-5, atol=1e-3)


def test_loss_goes_down():
    spec = configs.CONFIGS[1]
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    _, losses = H.run_oracle(spec, w, x, t, 30)
    assert losses[-1] < losses[0] and all(np.isfinite(losses))


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden vectors not generated yet")
def test_oracle_matches_reference_kernel_vectors():
    import sys
    sys.path.insert(0, os.path.dirname(GOLDEN))
    import make_golden
    gold = np.load(GOLDEN)
    checked = 0
    for spec, steps in make_golden.golden_specs():
        w = configs.make_weights(spec)
        x, t, _ = configs.make_data(spec)
        net, losses = H.run_oracle(spec, w, x, t, steps)
        np.testing.assert_allclose(losses, gold[f"{spec.name}/losses"], rtol=1e-5)
        mine = make_golden.digest([l.state() for l in net.layers], spec)
        for key, val in mine.items():
            if key.endswith("/mask"):
                assert np.array_equal(val, gold[key]), key
            elif val.size:
                assert H.relerr(val, gold[key]) <= 2e-5, key
            checked += 1
    assert checked > 100
