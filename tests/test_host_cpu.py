"""Host-side logic that needs no GPU: schedulers, ordinals, seeds, configs, init functions."""
import math

import numpy as np
import pytest

import soklyn_b200 as sk
from soklyn_b200 import configs
from soklyn_b200.function import Activation, LossFunc, Normalisation, Optimiser, Regularisation


def test_ordinals_are_the_kernel_abi():
    assert [a.ordinal() for a in (Activation.Identity, Activation.Sigmoid, Activation.ReLU, Activation.LeakyReLU(0.1),
                                  Activation.Tanh, Activation.Softmax, Activation.SiLU, Activation.Mish)] == list(range(8))
    assert [n.ordinal() for n in Normalisation] == [0, 1, 2, 3]
    assert Optimiser.SGD(0.9, True).ordinal() == 0 and Optimiser.Adam().ordinal() == 1
    assert [Regularisation.none().ordinal(), Regularisation.l1(0.1).ordinal(), Regularisation.l2(0.1).ordinal()] == [0, 1, 2]
    assert [l.value for l in LossFunc] == [0, 1, 2]
    assert Optimiser.SGD(0.9, True).kernel_args() == (0.9, 0.0, 0.0, 1)
    assert Optimiser.Adam(0.9, 0.999, 1e-8).kernel_args() == (0.9, 0.999, 1e-8, 0)


def test_cosine_decay_schedule():
    s = sk.CosineDecayLR(1e-5, 1e-3, 100, 10)
    assert s.get_learning_rate() == pytest.approx(1e-5)
    lrs = [s.step() for _ in range(100)]
    assert lrs[4] == pytest.approx(1e-5 + 0.5 * (1e-3 - 1e-5), rel=1e-6)     # warm-up is linear
    assert lrs[9] == pytest.approx(1e-3, rel=1e-6)                            # peak at the end of warm-up
    assert lrs[54] == pytest.approx(1e-5 + 0.5 * (1e-3 - 1e-5) * (1 + math.cos(math.pi * 45 / 90)), rel=1e-5)
    assert lrs[99] == pytest.approx(1e-5, abs=1e-9)
    assert all(a >= b for a, b in zip(lrs[9:], lrs[10:]))
    s.reset()
    assert s.get_learning_rate() == pytest.approx(1e-5)
    assert sk.CosineDecayLR(0.1, 0.5, 10, 10).step() == pytest.approx(0.1 + 0.1 * 0.4)
    z = sk.CosineDecayLR(0.1, 0.5, 5, 5)
    for _ in range(5):
        z.step()
    assert z.get_learning_rate() == pytest.approx(0.1)                        # decay_total == 0 -> min_lr


def test_exponential_and_plateau():
    e = sk.ExponentialLR(0.1, 0.5)
    assert [e.step(), e.step()] == pytest.approx([0.05, 0.025])
    e.reset()
    assert e.get_learning_rate() == pytest.approx(0.1)
    p = sk.ReduceLROnPlateauScheduler(2, sk.SchedulerMode.Minimize, 0.5, 0.02)
    p.reset(0.1)
    assert p.step(1.0) == pytest.approx(0.1)      # improvement
    assert p.step(1.0) == pytest.approx(0.1)      # 1 bad step
    assert p.step(2.0) == pytest.approx(0.05)     # patience reached
    assert p.step(float("nan")) == pytest.approx(0.05)
    assert p.step(3.0) == pytest.approx(0.05)
    assert p.step(3.0) == pytest.approx(0.025)
    assert p.step(3.0) == pytest.approx(0.025)
    assert p.step(3.0) == pytest.approx(0.02)     # clamped at min_lr
    m = sk.ReduceLROnPlateauScheduler(1, sk.SchedulerMode.Maximize, 0.1, 0.0)
    m.reset(1.0)
    assert m.step(0.5) == pytest.approx(1.0) and m.step(0.4) == pytest.approx(0.1)
    with pytest.raises(AssertionError):
        sk.ReduceLROnPlateauScheduler(0, sk.SchedulerMode.Minimize, 0.5, 0.0)


def test_scramble_seed_matches_native_and_oracle():
    from oracle import oracle as ok
    from soklyn_b200 import _native
    for step, lid in [(1, 0), (2, 23), (99, 54), (12345, 81)]:
        assert sk.scramble_seed(step, lid) == ok.scramble_seed(step, lid) == _native.lib().sk_scramble_seed(step, lid)


def test_config_recipes():
    c4 = configs.CONFIGS[4]
    assert c4.params() == 268_435_456
    assert c4.flops_per_step() == pytest.approx(12.09e12, rel=2e-3)
    assert configs.CONFIGS[1].flops_per_step() == pytest.approx(29.1e6, rel=5e-3)
    assert configs.CONFIGS[1].id_stride() == 23 and c4.id_stride() == 27
    x, t, labels = configs.make_data(configs.CONFIGS[1])
    assert x.shape == (64, 784) and t.shape == (64, 10) and (t.sum(1) == 1).all()
    assert np.allclose(x * 255, np.round(x * 255)) and x.min() >= 0 and x.max() <= 1
    w = configs.make_weights(configs.CONFIGS[1])
    assert abs(w[0].std() - math.sqrt(2 / 784)) < 2e-3
    x2, _, _ = configs.make_data(configs.CONFIGS[1])
    assert np.array_equal(x, x2)


def test_init_functions_have_the_reference_scales():
    n = 200_000
    assert abs(sk.InitHeNormalFunc(1).init(100, 50, n).std() - math.sqrt(2 / 100)) < 2e-3
    assert abs(sk.InitXavierNormalFunc(1).init(100, 50, n).std() - math.sqrt(2 / 150)) < 2e-3
    u = sk.InitXavierUniformFunc(1).init(100, 50, n)
    assert abs(np.abs(u).max() - math.sqrt(6 / 150)) < 1e-3 and abs(u.mean()) < 1e-3
    h = sk.InitHeUniformFunc(1, 0.5).init(100, 50, n)
    assert abs(np.abs(h).max() - 0.5 * math.sqrt(6 / 100)) < 1e-3
    assert (sk.InitZeroFunc().init(3, 3, 9) == 0).all()


def test_chacha8_block_function_known_answers():
    """The 8-round keystream of the all-zero key and nonce (the published ChaCha test vector for 8 rounds,
    256-bit key), and for comparison the 20-round one; the generator reads the same stream word by word."""
    from soklyn_b200.chacha import ChaCha8Rng, chacha_blocks
    zero = np.zeros(8, np.uint32)
    eight = chacha_blocks(zero, 0, 2, rounds=8)
    assert eight[0].astype("<u4").tobytes().hex() == (
        "3e00ef2f895f40d67f5bb8e81f09a5a12c840ec3ce9a7f3b181be188ef711a1e"
        "984ce172b9216f419f445367456d5619314a42a3da86b001387bfdb80e0cfe42")
    twenty = chacha_blocks(zero, 0, 1, rounds=20)
    assert twenty[0].astype("<u4").tobytes().hex().startswith("76b8e0ada0f13d90405d6ae55386bd28bdd219b8a08ded1aa836efcc8b770dc7")
    rng = ChaCha8Rng(zero)
    a, b = rng.next_u32s(21), rng.next_u32s(11)          # reads that straddle block boundaries
    assert np.array_equal(np.concatenate([a, b]), eight.reshape(-1))
    assert ChaCha8Rng(zero).next_u32() == int(eight[0, 0])


def test_seed_from_u64_is_deterministic_and_spreads_small_seeds():
    from soklyn_b200.chacha import seed_words_from_u64
    k0, k1 = seed_words_from_u64(0), seed_words_from_u64(1)
    assert np.array_equal(k0, seed_words_from_u64(0)) and not np.array_equal(k0, k1)
    assert len(set(k0.tolist())) == 8 and (k0 != 0).all()
    a = sk.InitHeNormalFunc(5).init(64, 32, 100)
    assert np.array_equal(a, sk.InitHeNormalFunc(5).init(64, 32, 100))
    two = sk.InitHeNormalFunc(5)
    first, second = two.init(64, 32, 60), two.init(64, 32, 40)      # the stream continues across calls
    assert np.array_equal(np.concatenate([first, second]), a)


def test_argmax_last_maximum_wins():
    from oracle import oracle as ok
    rows = np.array([[1, 3, 3, 0], [2, 2, 2, 2], [5, 1, 0, 0]], np.float32)
    assert ok.argmax_last(rows).tolist() == [2, 3, 0]


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(sk.log.DriverError):
        sk.GpuContext(16, 0)
