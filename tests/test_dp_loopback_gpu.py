"""The native data-parallel backward pass (sk_dp_backward) on ONE GPU: rank 0 of a two-rank job whose
other rank is a second arena in the same device's memory that contributes zero gradients and whose flag
words the host has raised beforehand. No kernel here waits for another kernel: every flag rank 0 polls is
already set, so the test exercises the row-block dW GEMMs, the exchange kernel (peer loads, optimiser step,
peer stores, flags), the column sums through the arena and the flag gate of the dX producer, and leaves the
real two-rank run to tests/test_dp_gpu.py.

With the peer's gradient zero the summed gradient is rank 0's own, averaged over twice the batch; Adam is
invariant to that factor (up to epsilon), so after one step the rows rank 0 owns must equal a plain one-GPU
step on the same batch under the 16-bit Adam rule of harness.compare_states, the rows it does not own must
be untouched, and the rows stored into the peer's weight tensor must equal rank 0's bit for bit. (One step
only: the silent peer never updates its rows, so later steps would see half-updated weights.)"""
import ctypes as C

import numpy as np
import pytest

import harness as H
from soklyn_b200 import configs
from soklyn_b200.configs import CONFIGS, scaled

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("blocks", [1, 2])
def test_native_dp_backward_as_rank0_against_a_silent_peer(gpu_ctx, blocks):
    import torch
    from soklyn_b200._native import SkExchange
    from soklyn_b200.core import Tensor, reset_tensor_ids
    from soklyn_b200.dp import _alias_tensor
    spec = scaled(CONFIGS[4], dims=(256, 512, 256, 512, 256), batch=192, name="dp_loopback")
    w = configs.make_weights(spec)
    x, t, _ = configs.make_data(spec)
    steps, world = 1, 2
    plain, _ = H.run_device(gpu_ctx, spec, w, x, t, steps)
    want = [H.device_state(gpu_ctx, l) for l in plain.get_layers()]

    net = H.build_device(gpu_ctx, spec, w)
    layers = net.get_layers()
    pad = lambda v: (v + 255) // 256 * 256
    offsets, total = [], 0
    for l in layers:
        nbytes = l.get_weights().rows() * l.get_weights().cols() * 2
        off = {"grad": total, "w": total + pad(nbytes)}
        off["flags"] = off["w"] + pad(nbytes)
        off["colsums"] = off["flags"] + pad(gpu_ctx.dp_flag_bytes())
        total = off["colsums"] + pad(3 * l.get_weights().cols() * 4)
        offsets.append(off)
    arenas = [gpu_ctx.peer_alloc(total)[0] for _ in range(world)]     # [0]: rank 0, [1]: the silent peer (all zero)
    try:
        flag_words = gpu_ctx.dp_flag_bytes() // 4
        for l, off in zip(layers, offsets):
            wt = l.get_weights()
            alias = _alias_tensor(arenas[0] + off["w"], tuple(wt.data.shape), wt.data.dtype, gpu_ctx.device)
            alias.copy_(wt.data)
            wt.data, l._desc = alias, None
            # the peer's flag words as rank 0 sees them: already beyond every epoch of this test
            flags = _alias_tensor(arenas[0] + off["flags"], (flag_words * 2,), torch.int16, gpu_ctx.device).view(torch.int32)
            flags.fill_(1000)
        tabs = (SkExchange * len(layers))()
        keep = []
        for i, off in enumerate(offsets):
            for name, field in (("grad", "peer_grad"), ("w", "peer_w"), ("flags", "peer_flags"), ("colsums", "peer_colsums")):
                arr = (C.c_void_p * world)(*[a + off[name] for a in arenas])
                keep.append(arr)
                setattr(tabs[i], field, C.cast(arr, C.c_void_p))
        xd = Tensor.from_cpu_vector(gpu_ctx, x, x.shape, spec.prec())
        td = Tensor.from_cpu_vector(gpu_ctx, t, t.shape, spec.prec())
        for s in range(1, steps + 1):
            net.forward(gpu_ctx, xd, spec.batch, False, s)
            gpu_ctx.gpu_dp_backward(layers, tabs, td, xd, spec.loss_config(), spec.train_context(), spec.batch, 2 * spec.batch,
                                    world, 0, blocks, s, s)
        gpu_ctx.synchronize()
        lr = spec.lr
        for i, (l, off, ref) in enumerate(zip(layers, offsets, want)):
            assert gpu_ctx.dp_blocks(l.get_weights().rows(), l.get_weights().cols(), world, blocks) == blocks
            got = H.device_state(gpu_ctx, l)
            # rows rank 0 owns: block c, first half of the block's rows; only they have current f32 masters
            k, p = l.get_weights().rows(), blocks
            own = np.zeros(k, bool)
            for c in range(p):
                own[c * (k // p): c * (k // p) + k // (p * world)] = True
            moved = np.abs(got["w"][own] - ref["w"][own]) / lr
            assert (moved > 0.1 * steps).mean() <= 0.01 and moved.max() <= 2.5 * steps, f"layer {i}: {moved.max():.2f} lr"
            assert np.array_equal(got["w"][~own], np.asarray(w[i], np.float32)[~own]), f"layer {i}: rows of the other rank changed"
            # the output block's delta is the plain run's; a hidden delta read the next layer's weights with only
            # rank 0's rows stepped (each step moves a weight by about lr, a percent of its size here)
            assert H.relerr(got["out"], ref["out"]) <= 2e-3
            delta_tol = 2e-3 if i == len(layers) - 1 else 5e-2
            assert H.relerr(got["d_prenorm"], ref["d_prenorm"]) <= delta_tol
            # bias: summed over both ranks' column sums (the peer's are zero) and averaged over twice the batch
            assert np.abs(got["b"] - ref["b"]).max() <= 2.5 * lr and H.relerr(got["dm_b"] * 2, ref["dm_b"]) <= delta_tol
            # the owned rows of the 16-bit weights landed in the peer's weight tensor as well, the others did not
            mine = l.get_weights().data
            peer = _alias_tensor(arenas[1] + off["w"], tuple(mine.shape), mine.dtype, gpu_ctx.device)
            own_t = torch.from_numpy(own).to(gpu_ctx.device)
            assert torch.equal(peer[own_t], mine[own_t]) and not bool(peer[~own_t].any())
            assert torch.equal(l.get_master_weights().data[own_t].to(mine.dtype), mine[own_t])
    finally:
        gpu_ctx.synchronize()
        for l in layers:      # the arenas go away: give the blocks ordinary storage back before they are freed
            wt = l.get_weights()
            wt.data, l._desc = wt.data.clone(), None
        for a in arenas:
            gpu_ctx.peer_free(a)
