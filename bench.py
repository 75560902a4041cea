#!/usr/bin/env python
"""Benchmark of the Q8_0 mul_mat hot path: the full LLaMA-3-8B decode matmul set at batch 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one token's worth of Q8_0 mul_mats: 32 layers x (q, k, v, o, gate, up, down) + lm_head =
225 matrices, 7.97 GB of Q8_0 weights streamed once.  With N > 1 (torchrun, one rank per GPU) every
weight is row-sharded over the ranks and each stage's output slices are all-gathered with NCCL.
Prints ONE JSON line (rank 0).  `--impl reference` times the reference's own CPU row-dot code
(oracle/_ref, built from the reference sources) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from nihilus_b200 import shapes, synth  # noqa: E402

METRIC = "q8_0_mul_mat_decode_set_hbm_gbs"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one full step (129 GEMV launches), from an ncu capture of one layer +
# lm_head scaled to 32 layers (every layer repeats the captured shapes): profiles/gemv_q8_rows_decode_set.md
NCU_DRAM_BYTES_PER_STEP = 8094.8e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.05):
        super().__init__(daemon=True)
        self.period = period
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def host_weights(layers_unique: int = 1):
    """Unique host tensors: one layer's seven projections + lm_head (other layers are row rotations)."""
    t0 = time.time()
    base = {}
    for name, (n, k) in shapes.LLAMA3_8B.items():
        base[name] = synth.make_weight(n, k, synth.seed_for(2, name, "weights"))
    return base, time.time() - t0


def cpu_reference_run(base, seconds_target: float, threads: int):
    """Times the reference's CPU row-dot code (oracle/_ref) or, if absent, the oracle port, on a bounded sample:
    layer-0's seven matrices + lm_head at batch 1, repeated until ~seconds_target of CPU work."""
    from oracle import pyoracle as po

    po.build()
    if po.Reference.available():
        impl, kind = po.Reference(), "reference"
        run = lambda w, x: impl.mul_mat(0, w, x, threads=threads)  # noqa: E731
    else:
        impl, kind = po.Oracle(), "port"
        run = lambda w, x: impl.mul_mat(po.Q8ACT_LANES, w, x, threads=threads)  # noqa: E731
    xs = {name: synth.make_activation(1, k, synth.seed_for(2, name, "activations")) for name, (n, k) in shapes.LLAMA3_8B.items()}
    nbytes = sum(shapes.mul_mat_bytes(n, k, 1) for n, k in shapes.LLAMA3_8B.values())
    run(base["attn_k"], xs["attn_k"])  # warm
    times = []
    t_end = time.time() + seconds_target
    while True:
        t0 = time.perf_counter()
        for name in shapes.LLAMA3_8B:
            run(base[name], xs[name])
        times.append(time.perf_counter() - t0)
        if time.time() >= t_end or len(times) >= 50:
            break
    return kind, nbytes, times


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    base, _ = host_weights()
    per_step_target = 2.0
    all_times = []
    kind, nbytes = "reference", 0
    for _ in range(args.warmup + args.steps):
        kind, nbytes, times = cpu_reference_run(base, per_step_target, threads)
        all_times.append(float(np.mean(times)))
        if len(all_times) >= 8:  # bounded: the whole arm stays within a few minutes
            break
    timed = all_times[min(args.warmup, len(all_times) - 1):]
    sec = float(np.mean(timed))
    value = nbytes / sec / 1e9
    sample = "layer-0 q,k,v,o,gate,up,down + lm_head at M=1 (790 MB of Q8_0 per pass), all host threads, row-partitioned"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": len(timed), "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "i8xi8->i32, f32 scales",
        "data": "synthetic",
        "config": {"workload": "configs[2]: LLaMA-3-8B full decode matmul set, batch 1 (bounded sample: 8 of 225 matrices per pass)",
                   "act_mode": "q8_0 activations"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def prefill_run(ctx, stream, torch, ops, weights, timed, world, M=512, iters=10):
    """configs[3]: a 512-token activation matrix times layer 0's gate, up and down weights (this rank's row shards).
    Returns whole-job TFLOP/s (2*M*N*K flops per mul_mat) and the fraction of the measured dense bf16 peak per GPU."""
    by_name = {}
    for i, (name, layer, n, k) in enumerate(ops):
        if layer == 0 and name in ("ffn_gate", "ffn_up", "ffn_down"):
            by_name[name] = (weights[i], n, k)
    if len(by_name) != 3:
        return None
    out = {}
    with torch.cuda.stream(stream):
        xs = {k: torch.randn((M, k), device="cuda") for k in {v[2] for v in by_name.values()}}
        ys = {name: torch.zeros((M, n), device="cuda") for name, (_, n, _) in by_name.items()}
    stream.synchronize()
    flops_total, ms_sum = 0, 0.0
    for name, (w, n, k) in by_name.items():
        fn = lambda: ctx.mul_mat(w, xs[k], ys[name])  # noqa: E731
        for _ in range(3):
            fn()
        ctx.sync()
        ms = timed(fn, iters) / iters
        out[name] = {"N": n, "K": k, "M": M, "ms": ms, "tflops": shapes.mul_mat_flops(n, k, M) / (ms * 1e-3) / 1e12}
        flops_total += shapes.mul_mat_flops(n, k, M)
        ms_sum += ms
    _, tf_peak, kind = measured_peaks()
    agg = flops_total / (ms_sum * 1e-3) / 1e12
    return {"workload": "configs[3]: M=512 x (gate, up 14336x4096; down 4096x14336), Q8_0 weights, Q8_0-quantised activations",
            "tflops": agg, "per_gpu_tflops": agg / world, "frac_of_bf16_peak": agg / world / tf_peak, "peak_tflops": tf_peak, "peak_kind": kind,
            "per_op": out, "note": "outside the timed decode region; weights of one layer (187 MB) exceed L2"}


def norm_run(ctx, stream, torch, ops, weights, timed, iters=20):
    """rms_norm x norm-weight, the producer of the q/k/v and gate/up activations (K = 4096): the kernel alone at 1 and
    512 rows, and one decode stage (norm -> q, k, v) as two calls against the fused call, rotating over the layers so
    the weights come from HBM when the rotation exceeds L2.  Every variant is captured into a CUDA graph first, like
    the decode step itself, so the figures are device time and not the host's launch rate."""
    K = shapes.LLAMA3_8B["attn_q"][1]
    by_layer = {}
    for i, (name, layer, n, k) in enumerate(ops):
        if name in ("attn_q", "attn_k", "attn_v"):
            by_layer.setdefault(layer, []).append((weights[i], n))
    layers = [v for _, v in sorted(by_layer.items()) if len(v) == 3][:8]
    hbm_peak, _, kind = measured_peaks()
    out = {"K": K, "eps": 1e-5, "sqrt_mode": "ieee"}

    def graph_us(fn, calls_per_fn):
        fn()  # first call outside the capture: scratch buffers are allocated here
        ctx.sync()
        ctx.graph_begin()
        fn()
        g = ctx.graph_end()
        for _ in range(3):
            g.launch()
        ctx.sync()
        ms = timed(g.launch, iters) / iters
        g.free()
        return ms * 1e3 / calls_per_fn

    with torch.cuda.stream(stream):
        nw = torch.rand(K, device="cuda") + 0.5
        for M in (1, 512):
            reps = 16
            xs = [torch.randn((M, K), device="cuda") for _ in range(reps)]
            y = torch.empty((M, K), device="cuda")
            us = graph_us(lambda: [ctx.rms_norm_mul(x, nw, 1e-5, y=y) for x in xs], reps)
            nbytes = 2 * M * K * 4 + K * 4
            out["rows_%d" % M] = {"us": us, "gbs": nbytes / (us * 1e-6) / 1e9, "frac_of_hbm_peak": nbytes / (us * 1e-6) / 1e9 / hbm_peak}
        if layers:
            x = torch.randn((1, K), device="cuda")
            ys = [[torch.zeros((1, n), device="cuda") for _, n in lw] for lw in layers]
            normed = torch.empty((1, K), device="cuda")

            def two_calls():
                for lw, ly in zip(layers, ys):
                    ctx.rms_norm_mul(x, nw, 1e-5, y=normed)
                    ctx.mul_mat_batch([(w, normed, yy) for (w, _), yy in zip(lw, ly)])

            def fused():
                for lw, ly in zip(layers, ys):
                    ctx.rms_norm_mul_mat_batch([(w, x, yy) for (w, _), yy in zip(lw, ly)], nw, 1e-5)

            def plain():
                for lw, ly in zip(layers, ys):
                    ctx.mul_mat_batch([(w, x, yy) for (w, _), yy in zip(lw, ly)])

            for name, fn in (("qkv_without_norm_us", plain), ("norm_then_qkv_two_calls_us", two_calls), ("norm_qkv_fused_us", fused)):
                out[name] = graph_us(fn, len(layers))
            out["stage_layers_in_rotation"] = len(layers)
    out["peak_kind"] = kind
    out["note"] = ("CUDA-graph replays; rows_1 and rows_512 are back-to-back launches of the kernel alone; the sum-of-squares chain is "
                   "K/8 = 512 dependent fma steps per row by the reference's definition")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=shapes.L, help="debug: fewer layers (the reported workload is 32)")
    ap.add_argument("--group", default="stage", choices=["stage", "op"], help="ops launched together: independent ops of a stage, or one by one")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--act-mode", default="q8", choices=["q8", "f32"],
                    help="q8: activations quantised to Q8_0, exact int8 block dots (the reported metric); f32: f32 activations x dequantised weights")
    ap.add_argument("--replicate-mb", type=int, default=48,
                    help="N > 1 placement policy: weights smaller than this many MiB stay whole on every rank (no exchange); 0 shards all")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl", "none"],
                    help="N > 1: outputs completed by the GEMV's own peer stores (fused) or by a grouped NCCL all-gather per stage")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 512-token GEMM and the rms_norm figures that ride along in the JSON line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from nihilus_b200 import build

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: nihilus_b200 has no CPU fallback")
    build.build()
    from nihilus_b200 import capi

    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    ctx = capi.Context(local, rank, world)
    if world > 1:
        ctx.set_option("replicate_below_mb", args.replicate_mb)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    if world > 1:
        uid = [capi.Context.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        ctx.comm_init(uid[0])

    # ---- data: synthetic, shapes and distributions of the LLaMA-3-8B Q8_0 model ----
    base, gen_s = host_weights()
    ops = shapes.decode_set(args.layers)
    weights = []
    t0 = time.time()
    for name, layer, n, k in ops:
        blocks = base[name] if layer <= 0 else synth.roll_rows(base[name], 17 * layer)
        weights.append(ctx.upload(blocks))
    upload_s = time.time() - t0
    x_off, y_off = [], []
    xo = yo = 0
    for name, layer, n, k in ops:
        x_off.append(xo)
        y_off.append(yo)
        xo += k
        yo += n
    x_host = torch.empty(xo, dtype=torch.float32).pin_memory()
    rng = np.random.default_rng(synth.seed_for(2, "attn_q", "activations"))
    x_host.numpy()[:] = rng.standard_normal(xo, dtype=np.float32)
    y_host = torch.empty(yo, dtype=torch.float32).pin_memory()
    with torch.cuda.stream(stream):
        x_dev = x_host.to("cuda", non_blocking=True)
        # with several ranks the outputs live in symmetric memory and the GEMV delivers every rank's columns itself
        y_dev = ctx.symm_empty((yo,)) if (world > 1 and args.gather == "fused") else torch.zeros(yo, dtype=torch.float32, device="cuda")
    stream.synchronize()
    xs = [x_dev[x_off[i]:x_off[i] + ops[i][3]].view(1, -1) for i in range(len(ops))]
    ys = [y_dev[y_off[i]:y_off[i] + ops[i][2]].view(1, -1) for i in range(len(ops))]

    # groups of independent ops: (q,k,v) (o) (gate,up) (down) per layer, then lm_head
    groups, i = [], 0
    if args.group == "stage":
        for layer in range(args.layers):
            for stage in shapes.LAYER_STAGES:
                groups.append(list(range(i, i + len(stage))))
                i += len(stage)
        groups.append([i])
    else:
        groups = [[j] for j in range(len(ops))]

    act_mode = capi.ACT_Q8 if args.act_mode == "q8" else capi.ACT_F32

    def enqueue_step():
        for g in groups:
            ctx.mul_mat_batch([(weights[j], xs[j], ys[j]) for j in g], act_mode=act_mode)
            if world > 1 and args.gather != "none":  # "none" leaves the rows incomplete: timing experiments only
                ctx.all_gather_batch([ys[j] for j in g])

    l0 = ctx.launches
    enqueue_step()  # eager once: allocations, attributes
    ctx.sync()
    launches_per_step = ctx.launches - l0
    graph = None
    if not args.no_graph:
        ctx.graph_begin()
        enqueue_step()
        graph = ctx.graph_end()

    def step():
        if graph is not None:
            graph.launch()
        else:
            enqueue_step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        ev0 = torch.cuda.Event(enable_timing=True)
        ev1 = torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(stream):
            ev0.record(stream)
            for _ in range(steps):
                fn()
            ev1.record(stream)
        ctx.sync()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(args.warmup):
        step()
    ctx.sync()
    sampler = ClockSampler(local)
    sampler.start()
    ms_total = timed(step, args.steps)
    clocks = sampler.stop()
    ms_step = ms_total / args.steps

    # ---- end to end: host activations in, host outputs out, through the C ABI every step ----
    x_bytes, y_bytes = xo * 4, yo * 4

    def e2e_step():
        ctx.memcpy_h2d(x_dev.data_ptr(), x_host.data_ptr(), x_bytes)
        step()
        ctx.memcpy_d2h(y_host.data_ptr(), y_dev.data_ptr(), y_bytes)

    for _ in range(3):
        e2e_step()
    ctx.sync()
    e2e_steps = max(10, args.steps // 4)
    e2e_ms = timed(e2e_step, e2e_steps) / e2e_steps

    total_bytes = sum(shapes.mul_mat_bytes(n, k, 1) for _, _, n, k in ops)
    weight_bytes = sum(n * (k // 32) * 34 for _, _, n, k in ops)
    value = total_bytes / (ms_step * 1e-3) / 1e9
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e9
    hbm_peak, _, peak_kind = measured_peaks()

    # ---- prefill (configs[3]): 512 tokens through layer 0's gate, up and down with the tensor-core GEMM ----
    prefill = None
    if not args.no_prefill:
        prefill = prefill_run(ctx, stream, torch, ops, weights, timed, world)

    # ---- rms_norm x norm-weight, the producer of the decode activations (1 GPU: it does not shard) ----
    norm = None
    if not args.no_prefill and world == 1 and args.act_mode == "q8":
        norm = norm_run(ctx, stream, torch, ops, weights, timed)

    # spot parity check of the timed buffers against nothing but themselves being finite (full parity lives in tests/)
    ctx.sync()
    finite = bool(torch.isfinite(y_dev).all().item())

    if rank == 0:
        gemv_launches = len(groups)
        per_launch_bytes = total_bytes / world / gemv_launches
        per_launch_ms = ms_step / gemv_launches
        per_gpu_gbs = total_bytes / world / (ms_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "i8xi8->i32, f32 scales", "data": "synthetic",
            "config": {
                "workload": "configs[2]: LLaMA-3-8B full decode matmul set, batch 1: %d layers x (q,k,v,o,gate,up,down) + lm_head = %d Q8_0 mul_mats, "
                            "%.3f GB of Q8_0 weights per step" % (args.layers, len(ops), weight_bytes / 1e9),
                "act_mode": "q8_0 activations (reference quantiser), exact int8 block dots" if args.act_mode == "q8" else "f32 activations x dequantised weights",
                "launch_grouping": args.group, "cuda_graph": graph is not None, "parallelism": "row-shard x%d" % world + ("" if world == 1 or not args.replicate_mb else " (weights under %d MiB replicated)" % args.replicate_mb) + ("" if world == 1 else (" + all-gather fused into the GEMV (peer stores over NVLink)" if args.gather == "fused" else " + NCCL all-gather per stage")),
                "l2": "inputs larger than L2 (%.2f GB of weights per GPU per step vs 126 MB)" % (weight_bytes / world / 1e9),
            },
            "tokens_per_s_equiv": 1e3 / ms_step,
            "frac_of_nominal_8TBs": per_gpu_gbs / NOMINAL_HBM_GBS,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_bytes, "d2h_bytes_per_step": y_bytes, "ms_per_step": e2e_ms},
            "gpu_launches": launches_per_step * args.steps,
            "launches_per_step": launches_per_step,
            "clocks": clocks,
            "roofline": {
                "bound": "hbm", "kernel": "gemv_q8_rows", "achieved": per_launch_bytes / (per_launch_ms * 1e-3) / 1e9, "peak": hbm_peak,
                "unit": "GB/s", "frac": per_launch_bytes / (per_launch_ms * 1e-3) / 1e9 / hbm_peak, "peak_kind": peak_kind,
                "traffic": (NCU_DRAM_BYTES_PER_STEP / gemv_launches) if (args.layers == shapes.L and world == 1) else None,
                "bytes_per_launch": per_launch_bytes, "ms_per_launch": per_launch_ms,
                "note": "per GPU; launch gaps inside the graph are included in the duration",
            },
            "prefill": prefill,
            "rms_norm": norm,
            "outputs_finite": finite,
            "setup_s": {"generate": gen_s, "upload": upload_s},
        }
        if world == 1 and not args.no_cpu_baseline:
            kind, nbytes, times = cpu_reference_run(base, args.cpu_seconds, os.cpu_count() or 1)
            line["cpu_baseline"] = {
                "value": nbytes / float(np.mean(times)) / 1e9, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": kind,
                "sample": "layer-0 q,k,v,o,gate,up,down + lm_head at M=1 (790 MB of Q8_0 per pass, %d passes), all host threads" % len(times),
            }
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)

    if graph is not None:
        graph.free()
    for w in weights:
        w.free()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
