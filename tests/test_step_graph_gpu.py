"""Whole-step CUDA graphs (sk_step_begin / sk_step_end, no counterpart in the reference): a training step
recorded and launched as one graph leaves every tensor bit-identical to the same step launched kernel by
kernel, although the step number, the learning rate and the dropout seed change from step to step."""
import numpy as np
import pytest

import harness as H
import soklyn_b200 as sk
from soklyn_b200 import configs
from soklyn_b200.configs import CONFIGS, scaled
from soklyn_b200.core import Tensor

pytestmark = pytest.mark.gpu

SPECS = [CONFIGS[1], CONFIGS[2],
         scaled(CONFIGS[3], dims=(384, 256, 128, 10), batch=96, name="classifier_small_dropout_cosine")]


@pytest.fixture(scope="module")
def gpu_ctx():
    ctx = sk.GpuContext(16, 0)
    yield ctx
    ctx.close()


def _train(ctx, spec, steps, slot):
    """`steps` training steps; slot None: kernel by kernel, else inside ctx.step_graph(slot)."""
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    net = H.build_device(ctx, spec, w, None)
    xd = Tensor.from_cpu_vector(ctx, x, x.shape, spec.prec())
    td = Tensor.from_cpu_vector(ctx, t, t.shape, spec.prec())
    lrs = H.lr_schedule(spec, steps)
    for s in range(1, steps + 1):
        tc = spec.train_context(lr=lrs[s - 1])
        if slot is None:
            outs = net.forward(ctx, xd, spec.batch, spec.use_dropout, s)
            net.backward(ctx, outs, td, xd, spec.loss_config(), tc, s)
        else:
            with ctx.step_graph(slot):
                outs = net.forward(ctx, xd, spec.batch, spec.use_dropout, s)
                net.backward(ctx, outs, td, xd, spec.loss_config(), tc, s)
    ctx.synchronize()
    return [H.device_state(ctx, l) for l in net.get_layers()]


@pytest.mark.parametrize("spec", SPECS, ids=lambda s: s.name)
def test_recorded_steps_equal_unrecorded_steps_bit_for_bit(gpu_ctx, spec):
    steps, slot = 7, SPECS.index(spec)
    want = _train(gpu_ctx, spec, steps, None)
    before = gpu_ctx.step_graph_stats()
    got = _train(gpu_ctx, spec, steps, slot)
    after = gpu_ctx.step_graph_stats()
    delta = {k: after[k] - before[k] for k in after}
    # the slot's first step runs unrecorded, the second instantiates the graph, the rest update it in place
    assert delta == {"unrecorded": 1, "instantiated": 1, "updated": steps - 2, "launched": steps - 1}, delta
    for i, (a, b) in enumerate(zip(got, want)):
        assert a.keys() == b.keys()
        for name in a:
            assert np.array_equal(a[name], b[name], equal_nan=True), f"layer {i} {name} differs under the step graph"


def test_two_networks_alternating_on_one_slot_reinstantiate_and_stay_correct(gpu_ctx):
    """A slot whose next step is another sequence of kernels cannot be updated in place: it is instantiated
    anew, and the results are still those of the unrecorded run."""
    a_spec, b_spec = CONFIGS[1], SPECS[2]
    want_a, want_b = _train(gpu_ctx, a_spec, 3, None), _train(gpu_ctx, b_spec, 3, None)
    before = gpu_ctx.step_graph_stats()
    got_a = _train(gpu_ctx, a_spec, 3, 5)     # slot 5: first use unrecorded, then recorded
    got_b = _train(gpu_ctx, b_spec, 3, 5)     # same slot, other network: all three recorded, first one re-instantiates
    after = gpu_ctx.step_graph_stats()
    assert after["instantiated"] - before["instantiated"] == 2
    assert after["launched"] - before["launched"] == 5
    for got, want in ((got_a, want_a), (got_b, want_b)):
        for a, b in zip(got, want):
            for name in a:
                assert np.array_equal(a[name], b[name], equal_nan=True), name


def test_waiting_inside_a_recorded_step_is_refused_and_the_context_stays_usable(gpu_ctx):
    spec = CONFIGS[1]
    want = _train(gpu_ctx, spec, 2, None)
    with gpu_ctx.step_graph(6):      # warms slot 6
        pass
    launched = gpu_ctx.step_graph_stats()["launched"]
    with pytest.raises(Exception, match="step graph is being recorded"):
        with gpu_ctx.step_graph(6):
            gpu_ctx.synchronize()    # refused; the context manager then drops the record
    assert gpu_ctx.step_graph_stats()["launched"] == launched
    with pytest.raises(Exception, match="without sk_step_begin"):
        gpu_ctx._check(gpu_ctx.lib.sk_step_end(gpu_ctx.handle))
    got = _train(gpu_ctx, spec, 2, 6)
    for a, b in zip(got, want):
        for name in a:
            assert np.array_equal(a[name], b[name], equal_nan=True), name
