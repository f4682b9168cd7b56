"""Data-parallel parity on real GPUs, run under torchrun (one rank per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 tests/dp_check.py

Every rank trains its row shard of a seeded batch for a few steps with DataParallelFFN; rank 0
also trains the whole batch on one device and requires the data-parallel weights, outputs and
dropout masks to agree with it (16-bit rule of tests/harness.py for Adam-updated parameters).
Exercised by tests/test_dp_gpu.py when two GPUs are visible."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import harness as H
    import soklyn_b200 as sk
    from soklyn_b200 import configs
    from soklyn_b200.core import Tensor, reset_tensor_ids
    from soklyn_b200.dp import DataParallelFFN
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = sk.GpuContext(16, local)
    steps = 3
    specs = [(configs.scaled(configs.CONFIGS[4], dims=(256, 512, 256, 512, 256), batch=256, name="dp_native_f16"), "native"),
             # per-rank batch above the row count from which the dX epilogue hands its column sums over, not a
             # multiple of the 32-row groups, with the statistics batch different from the local one
             (configs.scaled(configs.CONFIGS[4], dims=(128, 256, 128, 256, 128), batch=1100 * world, name="dp_native_tall_f16"), "native"),
             (configs.scaled(configs.CONFIGS[3], dims=(384, 256, 128, 16), batch=64 * world, name="dp_native_layernorm_dropout_f16"), "native"),
             # several tile columns per block of rows: the dX producer waits block by block
             (configs.scaled(configs.CONFIGS[4], dims=(1024, 2048, 1024), batch=1024 * world, name="dp_native_wide_f16"), "native"),
             (configs.scaled(configs.CONFIGS[4], dims=(128, 256, 128, 256, 128), batch=1100 * world, name="dp_fused_tall_f16"), "fused"),
             (configs.scaled(configs.CONFIGS[4], dims=(256, 512, 256, 512, 256), batch=256, name="dp_fused_f16"), "fused"),
             (configs.scaled(configs.CONFIGS[4], dims=(256, 512, 256, 512, 256), batch=256, name="dp_sharded_f16"), "sharded"),
             (configs.scaled(configs.CONFIGS[3], dims=(384, 256, 128, 16), batch=128, name="dp_dropout_layernorm_f16"), "auto"),
             (configs.scaled(configs.CONFIGS[1], dims=(96, 64, 32, 10), batch=64, name="dp_allreduce_f32"), "auto"),
             # BatchNorm: column statistics over the whole batch through the three-phase forward
             (configs.NetSpec(8, "dp_batchnorm_f32", (80, 64, 48, 12), ("batch", "batch", "disabled"),
                              ("tanh", "silu", "identity"), (0.0, 0.1, 0.0), "f32", "mse", "identity", "sgd", 0.05, 64,
                              "he_normal", "normal", "normal", True), "auto"),
             (configs.NetSpec(8, "dp_batchnorm_f16", (128, 256, 128, 16), ("batch", "rms", "disabled"),
                              ("silu", "silu", "identity"), (0.0, 0.0, 0.0), "f16", "mse", "identity", "adam", 1e-3, 128,
                              "xavier_normal", "normal", "normal"), "auto")]
    ok = True
    # the native exchange again in four blocks of rows (the dX producer waits block by block), and with the
    # arenas in symmetric memory (in-switch reduction and multicast stores where the node has them)
    variants = [(spec, scheme, {}) for spec, scheme in specs]
    variants += [(configs.scaled(spec, name=spec.name + "_blocks4"), "native", {"chunks": 4}) for spec, scheme in specs[:4]]
    variants += [(configs.scaled(spec, name=spec.name + "_multicast"), "native", {"multicast": "auto", "chunks": c})
                 for (spec, scheme), c in zip(specs[:4], (1, 4, 1, 4))]
    for spec, scheme, extra in variants:
        w = configs.make_weights(spec)
        x, t, _ = configs.make_data(spec)
        per = spec.batch // world
        reset_tensor_ids(0)
        net = configs.build_network(ctx, spec, w, max_batch=per)
        dp = DataParallelFFN(ctx, net, spec.batch, rank, world, scheme=scheme, **extra)
        xs = Tensor.from_cpu_vector(ctx, x[rank * per:(rank + 1) * per], (per, spec.dims[0]), spec.prec())
        ts = Tensor.from_cpu_vector(ctx, t[rank * per:(rank + 1) * per], (per, spec.dims[-1]), spec.prec())
        lrs = H.lr_schedule(spec, steps)
        for s in range(1, steps + 1):
            outs = dp.forward(xs, spec.use_dropout, s)
            dp.backward(outs, ts, xs, spec.loss_config(), spec.train_context(lr=lrs[s - 1]), s)
        ctx.synchronize()
        # every rank holds the same 16-bit / f32 weights afterwards
        for i, layer in enumerate(net.get_layers()):
            wt = layer.get_weights().data.float()
            ref = wt.clone()
            dist.broadcast(ref, 0)
            assert torch.equal(wt, ref), f"{spec.name}: layer {i} weights differ between ranks"
        dp.close()   # also completes the sharded masters and moments on every rank (gather_state)
        for i, layer in enumerate(net.get_layers()):
            for getter in ("get_master_weights", "get_dv_weights", "get_dm_weights"):
                state = getattr(layer, getter)()
                if state is None:
                    continue
                ref = state.data.clone()
                dist.broadcast(ref, 0)
                assert torch.equal(state.data, ref), f"{spec.name}: layer {i} {getter} differs between ranks after gather_state"
            if layer.get_master_weights() is not None:   # the 16-bit weights are the rounded masters, row for row
                assert torch.equal(layer.get_master_weights().data.to(layer.get_weights().data.dtype), layer.get_weights().data), \
                    f"{spec.name}: layer {i} weights are not the rounded master weights"
        if rank == 0:
            single, _ = H.run_device(ctx, spec, w, x, t, steps)
            tol = 1e-2 if spec.precision != "f32" else 5e-4
            for i, (a, b) in enumerate(zip(net.get_layers(), single.get_layers())):
                wa, wb = a.get_weights().download(ctx).astype(np.float64), b.get_weights().download(ctx).astype(np.float64)
                moved = np.abs(wa - wb) / max(lrs)
                rel = H.relerr(wa, wb)
                if spec.optimiser == "adam":
                    good = rel <= tol or ((moved > 0.1 * steps).mean() <= 0.02 and moved.max() <= 2.5 * steps)
                else:
                    good = rel <= tol
                oa, ob = a.get_outputs().download(ctx)[:per].astype(np.float64), b.get_outputs().download(ctx)[:per].astype(np.float64)
                rel_o = H.relerr(oa, ob)
                ma, mb = a.get_masks().download(ctx)[:per], b.get_masks().download(ctx)[:per]
                mask_ok = np.array_equal(ma != 0, mb != 0)
                print(f"{spec.name} L{i}: weights rel {rel:.2e} (max moved {moved.max():.2f} lr), outputs rel {rel_o:.2e}, "
                      f"masks {'equal' if mask_ok else 'DIFFER'}, exchange={dp.exchange_name()}, blocks={dp.blocks[i] if dp.blocks else 1}",
                      flush=True)
                ok = ok and good and mask_ok and rel_o <= 5 * tol
    flag = torch.tensor([1 if ok else 0], device=ctx.device)
    dist.broadcast(flag, 0)
    dist.destroy_process_group()
    if rank == 0:
        print("DP_CHECK_OK" if ok else "DP_CHECK_FAILED", flush=True)
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
