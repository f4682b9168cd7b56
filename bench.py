"""Benchmark of the DenseBlock / FeedForwardNetwork training step.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--config 4]

Workload (default): BASELINE config 4, the wide FFN 4096->16384->4096->16384->4096 in FP16
with FP32 masters, RMSNorm + SiLU, MSE, Adam, global batch 8192 split by rows across N
GPUs (strong scaling). One step = forward + backward + optimiser update of every layer.
Prints ONE JSON line (rank 0). Data are seeded synthetic tensors (soklyn_b200.configs).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the three GEMM classes of the
# default workload, from one ncu capture of this network at batch 2048 (a full-size capture would hold
# too much device memory for ncu's save/restore). Scaled to batch 8192 as: measured bytes + 3 x the bytes
# that grow with the batch (activations in and out of the GEMM and its epilogue); weights, and for dW the
# 26 B per parameter of the fused optimiser step, are the same at any batch. Averages over the launches
# of a class. These cannot be measured inside an unprofiled run, hence constants.
NCU_TRAFFIC_BYTES_PER_LAUNCH = {"gemm_forward": 545e6, "gemm_dx": 3017e6, "gemm_dw": 2166e6}


def measured_peaks():
    """Roofline denominators: the driver-written measurement of this pool's B200s when present."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops_burst": p["bf16_tflops"],
                "tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


def pick_peak(peaks, timed_seconds, clocks):
    """Which tensor peak a number is held against: the burst figure when the timed region was short and
    the SM clock stayed near its maximum (a kernel timed as if alone), else the sustained one."""
    sm, mx = (clocks or {}).get("sm_mhz"), (clocks or {}).get("sm_max_mhz")
    near_max = sm is not None and mx and sm >= 0.95 * mx
    if timed_seconds < 1.0 and near_max:
        return peaks["tflops_burst"], "burst"
    return peaks["tflops_sustained"], "sustained"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled during the timed region (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx, self.proc = device_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def timed_steps(step_fn, steps, warmup, world, device, before_timed=None):
    """W untimed steps, then K steps between barrier+synchronize, CUDA events, max over ranks (ms)."""
    import torch.distributed as dist
    for i in range(warmup):
        step_fn(i + 1)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    if before_timed is not None:
        before_timed()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(warmup + i + 1)
    e1.record()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def cpu_baseline_leg(spec, sample_rows: int):
    """The CPU oracle (a port: the reference has no CPU path) on `sample_rows` rows of the workload, one step."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import harness as H
    from soklyn_b200 import configs
    sample_rows = min(sample_rows, spec.batch)
    small = configs.scaled(spec, batch=sample_rows)
    w = configs.make_weights(small)
    x, t, _ = configs.make_data(small)
    net = H.build_oracle(small, w)
    opt = H._oracle_optim(small)
    steps, t0 = 0, time.perf_counter()
    while True:       # at least one step; small networks repeat until about two seconds have passed
        steps += 1
        outs = net.forward(x, small.batch, small.use_dropout, steps)
        net.backward(outs, t, x, small.loss, small.loss_act, opt, opt, small.batch, small.lr, steps)
        dt = time.perf_counter() - t0
        if dt > 2.0 or steps >= 2000:
            break
    cores = len(os.sched_getaffinity(0))
    return {"value": sample_rows * steps / dt, "unit": "samples/s", "cores": cores, "kind": "port",
            "sample": f"{steps} step(s) on {sample_rows} of {spec.batch} rows (OpenMP, {cores} threads), {dt:.1f} s"}


def multicast_choice(flag: str, world: int):
    """--dp-multicast auto (default): the in-switch reduction pays from eight GPUs on (3.10 against 3.36 ms per
    step; each GPU sends 134 MB per layer instead of 234 MB), so there the arenas go into symmetric memory when that
    can be set up; on two and four GPUs the plain peer loads and stores measured as fast or faster (7.50 against
    7.82 ms, 4.51 against 4.52) and stay. "on" / "off" force either."""
    if world <= 1 or flag == "off":
        return False
    if flag == "auto":
        return "auto" if world >= 8 else False
    return True


def run_ours(args):
    import torch.distributed as dist
    import soklyn_b200 as sk
    from soklyn_b200 import configs
    from soklyn_b200.core import Tensor
    from soklyn_b200.dp import DataParallelFFN
    rank, local_rank, world = dist_env()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    spec = configs.CONFIGS[args.config]
    if args.batch:
        spec = configs.scaled(spec, batch=args.batch)
    if args.lr > 0:
        from dataclasses import replace
        spec = replace(spec, lr=args.lr)
    ctx = sk.GpuContext(16, local_rank)
    if args.lean:
        ctx.set_lean_backward(True)
    local = spec.batch // world
    net = configs.build_network(ctx, spec, max_batch=local)
    dp = DataParallelFFN(ctx, net, spec.batch, rank, world, scheme=args.dp_scheme, chunks=args.dp_chunks,
                         multicast=multicast_choice(args.dp_multicast, world))
    x, t, _ = configs.make_data(spec)
    r0 = rank * local
    prec = spec.prec()
    tdt = torch.float16 if spec.precision == "f16" else torch.float32
    x_host = torch.from_numpy(x[r0:r0 + local]).to(tdt).pin_memory()
    t_host = torch.from_numpy(t[r0:r0 + local]).to(tdt).pin_memory()
    xd = Tensor.from_cpu_vector(ctx, x_host, x_host.shape, prec)
    td = Tensor.from_cpu_vector(ctx, t_host, t_host.shape, prec)
    tc = spec.train_context()
    lc = spec.loss_config()

    # Whole-step CUDA graphs for the launch-bound small networks (configs 1-3 on one GPU); the wide FFN's 23
    # launches per 13 ms step gain nothing from them and stay kernel by kernel.
    use_graph = world == 1 and (args.step_graph == "on" or (args.step_graph == "auto" and spec.cfg in (1, 2, 3)))

    def step_eager(s):
        outs = dp.forward(xd, spec.use_dropout, s)
        dp.backward(outs, td, xd, lc, tc, s)

    def step_resident(s):
        if use_graph:
            with ctx.step_graph(0):
                step_eager(s)
        else:
            step_eager(s)

    out_host = [torch.empty((local, spec.dims[-1]), dtype=tdt).pin_memory() for _ in range(2)]
    from soklyn_b200.pipeline import HostFeeder
    feeder = HostFeeder(ctx, [tuple(x_host.shape), tuple(t_host.shape)], prec)
    feeder.stage(1, [x_host, t_host])   # the first step (s = 1) reads slot 1

    def step_e2e(s):
        # inputs of this step were staged from pinned host memory during the previous one; the next step's
        # are staged now; the output goes back to the host while backward runs, into one of two host
        # buffers, and the host waits for it only after the NEXT step has been queued (every step's result
        # is read; the device never idles while the host waits)
        slot = s % 2
        xs, ts = feeder.acquire(slot)
        feeder.stage(1 - slot, [x_host, t_host])
        outs = dp.forward(xs, spec.use_dropout, s)
        feeder.fetch(outs[-1], out_host[slot], local, slot)
        dp.backward(outs, ts, xs, lc, tc, s)
        feeder.release(slot)
        feeder.wait_output(1 - slot)                # the previous step's result is on the host

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = [0]

    def arm():   # runs after the warm-up
        launches0[0] = ctx.launch_count()

    ms = timed_steps(step_resident, args.steps, args.warmup, world, device, before_timed=arm)
    launches = ctx.launch_count() - launches0[0]
    clocks = sampler.stop() if rank == 0 else None
    eager_ms = timed_steps(step_eager, args.steps, 2, world, device) if use_graph else None
    # Per-kernel-class device times come from CUDA events around every launch; they are taken in a
    # second pass of the same K steps so that the event records stay out of the timed region.
    ctx.profile_enable(True)
    for i in range(args.steps):
        step_resident(args.warmup + args.steps + i + 1)
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    # the e2e warm-up must leave slot parity consistent: step numbers continue from the warm-up
    ms_e2e = timed_steps(step_e2e, args.steps, 2, world, device)
    # the same K steps once more with the lean backward option (not the headline: it leaves four API-visible
    # gradient tensors of the hidden blocks unwritten), so that the line carries both
    lean_ms = None
    if world == 1 and spec.cfg == 4 and not args.lean:
        ctx.set_lean_backward(True)
        lean_ms = timed_steps(step_resident, args.steps, 2, world, device)
        ctx.profile_enable(True)
        for i in range(args.steps):
            step_resident(10 ** 5 + i)
        lean_prof = ctx.profile_read()
        ctx.profile_enable(False)
        ctx.set_lean_backward(False)

    # Correctness carried in the line: the loss of one more forward pass on the resident inputs (the
    # same host formula on every rank's rows, averaged), and under data parallelism the largest
    # difference between any rank's weights and rank 0's, which must be zero.
    outs = dp.forward(xd, False, 10 ** 6)
    ctx.synchronize()
    diff = (outs[-1].data[:local].float() - td.data[:local].float())
    loss_t = (0.5 * (diff * diff).mean() if spec.loss == "mse" else torch.zeros((), device=device)).reshape(1).double()
    w_diff = torch.zeros(1, device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(loss_t)
        loss_t /= world
        for layer in net.get_layers():
            wt = layer.get_weights().data.float()
            ref0 = wt.clone()
            dist.broadcast(ref0, 0)
            w_diff = torch.maximum(w_diff, (wt - ref0).abs().max().double().reshape(1))
        dist.all_reduce(w_diff, op=dist.ReduceOp.MAX)
    loss_after, w_diff = float(loss_t.item()), float(w_diff.item())

    if rank == 0:
        peaks = measured_peaks()
        per_step = ms / args.steps
        gemm = {k: v for k, v in prof.items() if k.startswith("gemm")}
        top = max(gemm, key=lambda k: gemm[k][1])
        m_local = local
        flops = {"gemm_forward": sum(2.0 * m_local * spec.dims[i] * spec.dims[i + 1] for i in range(spec.layers)),
                 "gemm_dw": sum(2.0 * m_local * spec.dims[i] * spec.dims[i + 1] for i in range(spec.layers)),
                 "gemm_dx": sum(2.0 * m_local * spec.dims[i] * spec.dims[i + 1] for i in range(1, spec.layers))}
        n_l, t_ms = gemm[top]
        achieved = flops[top] * args.steps / (t_ms * 1e-3) / 1e12 if t_ms > 0 else 0.0
        peak, peak_kind = pick_peak(peaks, ms * 1e-3, clocks)
        per_class = {k: {"tflops": flops[k] * args.steps / (v[1] * 1e-3) / 1e12, "frac_burst": flops[k] * args.steps / (v[1] * 1e-3) / 1e12 / peaks["tflops_burst"],
                         "frac_sustained": flops[k] * args.steps / (v[1] * 1e-3) / 1e12 / peaks["tflops_sustained"]}
                     for k, v in gemm.items() if v[1] > 0}
        line = {
            "metric": "FFN train samples/s", "value": spec.batch / (per_step * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": spec.precision, "data": "synthetic (seeded N(0,1) inputs/targets, Xavier-uniform weights)",
            "config": {"workload": spec.name, "global_batch": spec.batch, "parallelism": f"dp{world}", "exchange": dp.exchange_name(),
                       "params": spec.params(), "lean": bool(args.lean), "step_graph": bool(use_graph),
                       "l2": "working set per step is far larger than L2 (126 MB)"},
            "tflops_per_step": spec.flops_per_step() / 1e12,
            "tflops_achieved": spec.flops_per_step() / (per_step * 1e-3) / 1e12,
            "e2e": {"value": spec.batch / (ms_e2e / args.steps * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": (x_host.numel() + t_host.numel()) * x_host.element_size(),
                    "d2h_bytes_per_step": out_host[0].numel() * out_host[0].element_size()},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak,
                         "frac_burst": achieved / peaks["tflops_burst"], "frac_sustained": achieved / peaks["tflops_sustained"],
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get(top) if spec.cfg == 4 and world == 1 and not args.batch else None,
                         "traffic_note": "bytes per launch: ncu capture at batch 2048, batch-proportional part scaled to 8192",
                         "peak_source": f"{peaks['source']} bf16 matmul, {peak_kind} (timed region {ms * 1e-3:.2f} s)",
                         "launches": int(n_l), "ms_per_launch": t_ms / max(1, n_l), "per_class": per_class},
            "kernel_ms_per_step": {k: v[1] / args.steps for k, v in prof.items()},
            "loss_after": loss_after,
        }
        if eager_ms is not None:
            line["step_graph"] = {"ms_per_step": per_step, "kernel_by_kernel_ms_per_step": eager_ms / args.steps, **ctx.step_graph_stats(),
                                  "note": "every step recorded by stream capture and launched as one graph (sk_step_begin / sk_step_end)"}
        if lean_ms is not None:
            line["lean"] = {"ms_per_step": lean_ms / args.steps, "value": spec.batch / (lean_ms / args.steps * 1e-3), "unit": "samples/s",
                            "gemm_dx_ms_per_step": lean_prof["gemm_dx"][1] / args.steps,
                            "gemm_dx_tflops": flops["gemm_dx"] * args.steps / (lean_prof["gemm_dx"][1] * 1e-3) / 1e12,
                            "note": "SK_OPTION_LEAN_BACKWARD: hidden blocks skip the stores of grad, f32 d_prenorm, d_norm_w, d_norm_b"}
        if world > 1:
            line["dp_check"] = {"max_abs_weight_diff_vs_rank0": w_diff, "loss_after": loss_after,
                                "note": "every rank's 16-bit weights compared with rank 0's after the timed steps; "
                                        "loss of one more forward pass over the whole batch"}
        if world == 1 and spec.cfg == 4 and not args.no_gemm_sweep:
            line["dense_block_gemm"] = gemm_sweep_rows(ctx, [16384], [1024, 4096, 8192], ["f16"], peaks)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg(spec, args.cpu_rows)
        print(json.dumps(line), flush=True)
    dp.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def gemm_sweep_rows(ctx, ms_list, kn_list, dtypes, peaks, index0: int = 0):
    """The three GEMMs of one DenseBlock in isolation, with their fused epilogues, over M x K x N: forward
    with bias + activation, dX with the activation-derivative / mask epilogue, dW with the column sums and
    the fused optimiser step. X, W, dY ~ N(0,1)/sqrt(K), seeded. One record per (dtype, M, K, N)."""
    import soklyn_b200 as sk
    from soklyn_b200.configs import _GivenWeights
    from soklyn_b200.core import Tensor
    acts = [sk.Activation.ReLU, sk.Activation.SiLU, sk.Activation.Tanh]
    rows, idx = [], index0
    for prec_name in dtypes:
        # "f32tc": f32 blocks with SK_OPTION_F32_TENSOR_CORES (three bf16 parts per operand in the workspace)
        prec = {"f16": sk.Precision.FP16, "f32": sk.Precision.FP32, "f32tc": sk.Precision.FP32, "bf16": sk.Precision.BF16}[prec_name]
        ctx.set_f32_tensor_cores(prec_name == "f32tc")
        if prec_name == "f32tc":
            ctx.reserve(6 * 2 * max(max(ms_list), max(kn_list)) * max(kn_list) + (1 << 20))   # both operands of the largest product, three bf16 parts each
        for m in ms_list:
            for k in kn_list:
                for n in kn_list:
                    gen = torch.Generator(device="cpu").manual_seed(5000 + idx)
                    act = acts[idx % 3]
                    idx += 1
                    w = (torch.randn(k, n, generator=gen) / k ** 0.5).numpy()
                    cfg = sk.LayerInitConfig(sk.Normalisation.Disabled, act, sk.Regularisation.none(), 0.0)
                    blk = sk.DenseBlock(ctx, True, k, n, m, _GivenWeights(w), cfg, prec)
                    nxt = sk.DenseBlock(ctx, True, n, k, m, _GivenWeights(w.T.copy()), sk.LayerInitConfig(), prec)
                    x = Tensor.from_cpu_vector(ctx, (torch.randn(m, k, generator=gen) / k ** 0.5).numpy(), (m, k), prec)
                    dy = torch.randn(m, k, generator=gen) / k ** 0.5
                    nxt.get_delta_prenorm_out().data.copy_(dy)
                    if nxt.d_prenorm_lp is not None:
                        nxt.d_prenorm_lp.data.copy_(dy)
                    tc = sk.TrainContext(sk.Optimiser.Adam(), sk.Optimiser.Adam(), m, 1e-3)
                    ops = {"forward": lambda: blk.forward(ctx, x, m, False, 1),
                           "dX": lambda: ctx.gpu_hidden_layer_error(blk, nxt, m),
                           "dW": lambda: ctx.gpu_backward_pass(blk, x, tc, 1)}
                    rec = {"dtype": prec_name, "M": m, "K": k, "N": n, "act": act.ordinal()}
                    heavy = float(m) * k * n >= 1e12 or (prec_name.startswith("f32") and float(m) * k * n > 2e11)
                    for name, fn in ops.items():
                        for _ in range(1 if heavy else 3):
                            fn()
                        torch.cuda.synchronize()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        iters = 2 if heavy else 5
                        e0.record()
                        for _ in range(iters):
                            fn()
                        e1.record()
                        torch.cuda.synchronize()
                        ms = e0.elapsed_time(e1) / iters
                        rec[name + "_ms"] = round(ms, 4)
                        rec[name + "_tflops"] = round(2.0 * m * k * n / (ms * 1e-3) / 1e12, 1)
                    rows.append(rec)
                    del blk, nxt, x
                    torch.cuda.empty_cache()
    ctx.set_f32_tensor_cores(False)
    sixteen = [r for r in rows if not r["dtype"].startswith("f32")]
    out = {"metric": "DenseBlock GEMM TFLOP/s", "unit": "TFLOP/s", "shapes": rows,
           "timing": "CUDA events around back-to-back calls of one entry point after warm-up; every call streams "
                     "operands and epilogue tensors larger than L2 for M >= 4096"}
    if sixteen:
        mean = sum(r["forward_tflops"] + r["dX_tflops"] + r["dW_tflops"] for r in sixteen) / (3 * len(sixteen))
        out.update({"mean_16bit": mean, "frac_burst": mean / peaks["tflops_burst"], "frac_sustained": mean / peaks["tflops_sustained"],
                    "best_forward": max(r["forward_tflops"] for r in sixteen)})
    return out


def run_gemm_sweep(args):
    """BASELINE config 5: the whole M x K x N sweep in both precisions, one JSON line."""
    import soklyn_b200 as sk
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    ctx = sk.GpuContext(16, 0)
    peaks = measured_peaks()
    ms_list = [int(v) for v in args.sweep_m.split(",")]
    kn_list = [int(v) for v in args.sweep_kn.split(",")]
    res = gemm_sweep_rows(ctx, ms_list, kn_list, args.sweep_dtypes.split(","), peaks)
    rows = res["shapes"]
    big = [r for r in rows if not r["dtype"].startswith("f32") and r["M"] >= 4096]
    best = max((r["forward_tflops"] for r in big), default=0.0)
    mean = sum(r["forward_tflops"] + r["dX_tflops"] + r["dW_tflops"] for r in big) / max(1, 3 * len(big))
    f32 = [r for r in rows if r["dtype"] == "f32" and r["M"] >= 4096]
    mean32 = sum(r["forward_tflops"] + r["dX_tflops"] + r["dW_tflops"] for r in f32) / max(1, 3 * len(f32))
    line = {"metric": "DenseBlock GEMM TFLOP/s", "value": mean, "unit": "TFLOP/s", "n_gpus": 1, "steps": 1, "warmup": 3,
            "higher_is_better": True, "dtype": args.sweep_dtypes, "data": "synthetic (seeded N(0,1)/sqrt(K))",
            "config": {"workload": "dense_block_gemm_sweep", "M": ms_list, "KN": kn_list,
                       "note": "value = mean over forward/dX/dW of the 16-bit cases with M >= 4096, fused epilogues included"},
            "best_forward_tflops": best, "peak_burst": peaks["tflops_burst"], "peak_sustained": peaks["tflops_sustained"],
            "frac_burst": mean / peaks["tflops_burst"], "frac_sustained": mean / peaks["tflops_sustained"],
            "mean_f32_tflops": mean32, "sweep": rows}
    # the wide shapes (K, N >= 4096) apart: the narrow ones are bound by the epilogue's HBM traffic, not by the tensor pipe
    wide = [r for r in big if r["K"] >= 4096 and r["N"] >= 4096]
    if wide:
        per = {k: sum(r[k + "_tflops"] for r in wide) / len(wide) for k in ("forward", "dX", "dW")}
        wmean = sum(per.values()) / 3
        line["wide_shapes"] = {"K_N_at_least": 4096, "mean_tflops": wmean, "frac_burst": wmean / peaks["tflops_burst"],
                               "frac_sustained": wmean / peaks["tflops_sustained"], "per_class_tflops": per}
    f32tc = [r for r in rows if r["dtype"] == "f32tc" and r["M"] >= 4096]
    if f32tc:
        line["mean_f32_tensor_core_tflops"] = sum(r["forward_tflops"] + r["dX_tflops"] + r["dW_tflops"] for r in f32tc) / (3 * len(f32tc))
    print(json.dumps(line), flush=True)
    ctx.close()


def run_reference(args):
    """The reference's own kernels (oracle/_ref: its unmodified nn_math.cu, JIT-ed from compute_75 PTX as its
    build.rs targets) with its launch configuration and its stream synchronisation after every launch, on
    the whole batch of the workload, on ONE GPU (the reference is single-device): rank 0 runs, other ranks
    leave. The reference has no CPU implementation of this path (every operation is a CUDA launch), so this is
    its stock code path. The process loads oracle/_ref/libsoklyn_ref.so and not the product library; the
    Python classes that sequence the layers are the host mirror of the reference's DenseBlock /
    FeedForwardNetwork. Falls back to the CPU port of the reference when oracle/_ref is absent."""
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    from soklyn_b200 import configs
    spec = configs.CONFIGS[args.config if args.config in configs.CONFIGS else 4]
    if args.batch:
        spec = configs.scaled(spec, batch=args.batch)
    rows = args.ref_rows if args.ref_rows > 0 else spec.batch
    sample = configs.scaled(spec, batch=rows)
    from oracle import ref_kernels
    if not ref_kernels.available() or not torch.cuda.is_available():
        cb = cpu_baseline_leg(spec, args.cpu_rows)
        line = {"impl": "reference", "metric": "FFN train samples/s", "value": cb["value"], "unit": "samples/s",
                "n_gpus": 1, "steps": 1, "warmup": 0, "ms_per_step": 1e3 * args.cpu_rows / cb["value"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": {"workload": spec.name, "global_batch": spec.batch},
                "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "samples/s", "h2d_bytes_per_step": 0,
                                            "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return
    from soklyn_b200.core import Tensor, reset_tensor_ids
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    ctx = ref_kernels.RefContext(16, local_rank, sync_each_launch=True)
    w = configs.make_weights(sample)
    x, t, _ = configs.make_data(sample)
    reset_tensor_ids(0)
    net = configs.build_network(ctx, sample, w)
    xd = Tensor.from_cpu_vector(ctx, x, x.shape, sample.prec())
    td = Tensor.from_cpu_vector(ctx, t, t.shape, sample.prec())
    tc, lc = sample.train_context(), sample.loss_config()

    def step(s):
        outs = net.forward(ctx, xd, rows, sample.use_dropout, s)
        net.backward(ctx, outs, td, xd, lc, tc, s)

    l0 = [0]

    def arm():
        l0[0] = ctx.ref_launch_count()

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed_steps(step, args.steps, args.warmup, 1, device, before_timed=arm)
    clocks = sampler.stop()
    per_step = ms / args.steps
    val = rows / (per_step * 1e-3)
    line = {"impl": "reference", "metric": "FFN train samples/s", "value": val, "unit": "samples/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": spec.precision, "data": "synthetic",
            "config": {"workload": spec.name, "global_batch": spec.batch, "rows_per_step": rows, "parallelism": "dp1",
                       "note": "the reference is single-device: one GPU whatever --gpus says"},
            "gpu_launches": int(ctx.ref_launch_count() - l0[0]), "clocks": clocks,
            "cpu_baseline": {"value": val, "unit": "samples/s", "cores": 1, "kind": "reference",
                             "sample": f"the reference's own CUDA kernels (it has no CPU path) on one B200, one host "
                                       f"thread, all {rows} rows per step, synchronising after every launch"},
            "e2e": {"value": val, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=4)
    ap.add_argument("--batch", type=int, default=0, help="override the global batch (parity/debug runs)")
    ap.add_argument("--cpu-rows", type=int, default=256, help="rows of the batch the CPU baseline leg runs")
    ap.add_argument("--ref-rows", type=int, default=0,
                    help="rows of the batch the reference arm runs per step (0: the whole batch)")
    ap.add_argument("--lr", type=float, default=0.0, help="override the configuration's learning rate")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gemm-sweep", action="store_true", help="leave the M = 16384 DenseBlock GEMM shapes out of the line")
    ap.add_argument("--lean", action="store_true", help="SK_OPTION_LEAN_BACKWARD (not the headline configuration)")
    ap.add_argument("--dp-multicast", default="auto", choices=["auto", "on", "off"],
                    help="exchange arena in symmetric memory: in-switch reduction and multicast stores where the node has them")
    ap.add_argument("--dp-chunks", type=int, default=0, help="row blocks per layer of the native exchange (0: one)")
    ap.add_argument("--dp-scheme", default="auto", choices=["auto", "native", "fused", "sharded", "allreduce"],
                    help="gradient exchange of the data-parallel runs (see soklyn_b200/dp.py)")
    ap.add_argument("--sweep-m", default="256,1024,4096,16384,65536")
    ap.add_argument("--sweep-kn", default="1024,4096,8192")
    ap.add_argument("--step-graph", choices=["auto", "on", "off"], default="auto",
                    help="launch each training step as one CUDA graph (auto: configs 1-3 on one GPU)")
    ap.add_argument("--sweep-dtypes", default="f16,f32", help="comma list of f16, bf16, f32, f32tc (f32 with the tensor-core option)")
    args = ap.parse_args()
    if args.config == 5 and args.impl != "reference":
        run_gemm_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
