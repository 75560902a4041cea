#!/usr/bin/env python
"""Benchmark of the Q8_0 mul_mat hot path: the full LLaMA-3-8B decode matmul set at batch 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one token's worth of Q8_0 mul_mats: 32 layers x (q, k, v | o | gate, up | down) + lm_head =
225 matrices in 129 stages (one launch each, in stream order), 7.97 GB of Q8_0 weights streamed once.  The independent
projections of a stage share one launch and one input vector (q/k/v read the same normalised row, gate/up likewise, as in
the reference's graph: include/nihilus-incl/infra/core_traits.hpp:575-594, 976-980); every stage reads its own synthetic
N(0,1) vector.  With N > 1 (torchrun, one rank per GPU) the larger weights are row-sharded over the ranks and every
stage's output slices are delivered to all ranks; the step ends with a wait for every delivery, launches in between wait
for the other ranks only where they read delivered rows (none do here: `every_launch_waits_ms_per_step` is the same step
with every launch waiting).  Prints ONE JSON line (rank 0).  `--impl reference` times the reference's own CPU
row-dot code (oracle/_ref, built from the reference sources) on the host cores instead, on the same 225 matrices.
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
DTYPE = "i8xi8->i32, f32 scales"
# dram__bytes_read.sum + dram__bytes_write.sum of one full step (129 GEMV launches), from an ncu capture of one layer +
# lm_head scaled to 32 layers (every layer repeats the captured shapes): profiles/gemv_q8_rows_decode_set.md
NCU_DRAM_BYTES_PER_STEP = 8152.0e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML every few milliseconds; `window` picks the samples that fell
    inside the timed region."""

    def __init__(self, index: int, period: float = 0.002):
        super().__init__(daemon=True)
        self.period = period
        self.samples: list[tuple[float, int]] = []
        self.reasons: list[tuple[float, str]] = []
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
                now = time.perf_counter()
                self.samples.append((now, int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.append((now, name))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)

    def window(self, t0: float, t1: float):
        inside = [mhz for t, mhz in self.samples if t0 <= t <= t1]
        return {"sm_mhz": int(np.median(inside)) if inside else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted({n for t, n in self.reasons if t0 <= t <= t1}), "samples": len(inside),
                "sampling": "NVML every %.0f ms; samples taken between the start and the end of the timed region" % (self.period * 1e3)}


def host_weights():
    """Unique host tensors: one layer's seven projections + lm_head (other layers are row rotations)."""
    t0 = time.time()
    base = {}
    for name, (n, k) in shapes.LLAMA3_8B.items():
        base[name] = synth.make_weight(n, k, synth.seed_for(2, name, "weights"))
    return base, time.time() - t0


def layer_weight(base, name, layer):
    return base[name] if layer <= 0 else synth.roll_rows(base[name], 17 * layer)


# ---------------------------------------------------------------------------------------------------------------
# CPU legs: the reference's own row-dot code (oracle/_ref) or, where it could not be built, the oracle port.
# The only place in this file that touches oracle/.
# ---------------------------------------------------------------------------------------------------------------
class CpuSet:
    """The decode set on the host: every one of the 225 matrices materialised (rows rotated per layer exactly as the GPU
    upload does) when the machine has the memory for it, otherwise layer 0's matrices stand in for every layer."""

    def __init__(self, base, layers: int):
        from oracle import pyoracle as po

        po.build()
        if po.Reference.available():
            self.impl, self.kind = po.Reference(), "reference"
            self.q8_mode = 0
        else:
            self.impl, self.kind = po.Oracle(), "port"
            self.q8_mode = po.Q8ACT_LANES
        self.po = po
        self.ops = shapes.decode_set(layers)
        need = sum(n * (k // 32) * 34 for _, _, n, k in self.ops)
        try:
            import psutil

            avail = psutil.virtual_memory().available
        except Exception:
            avail = 0
        self.distinct = avail > need + (6 << 30)
        self.mats = []
        for name, layer, n, k in self.ops:
            self.mats.append(layer_weight(base, name, layer) if self.distinct else base[name])
        self.xs = {k: synth.make_activation(1, k, synth.seed_for(2, "attn_q", "activations") + k) for k in {k for _, _, _, k in self.ops}}
        self.nbytes = sum(shapes.mul_mat_bytes(n, k, 1) for _, _, n, k in self.ops)

    def run(self, w, x, threads):
        return self.impl.mul_mat(self.q8_mode, w, x, threads=threads)

    def step(self, threads: int) -> float:
        t0 = time.perf_counter()
        for (name, layer, n, k), w in zip(self.ops, self.mats):
            self.run(w, self.xs[k], threads)
        return time.perf_counter() - t0

    def describe(self, threads):
        return ("all %d matrices of the set at M=1 (%.2f GB of Q8_0 per pass; %s), %d host threads, row-partitioned" %
                (len(self.ops), self.nbytes / 1e9, ("%d distinct host copies" % len(self.ops)) if self.distinct else "layer 0's matrices reused for every layer: not enough host memory for a copy of each", threads))


def cpu_baseline_leg(base, layers, seconds_target: float, gpu_check=None):
    """Bounded CPU sample for the repo arm's JSON line (N = 1, rank 0): the full set on all host threads, a one-thread leg
    on layer 0 + lm_head (how the reference's eval dispatcher ran it, cpu/avx_2.hpp:4983-4984), a 512-token prefill
    leg, and -- the oracle as checker -- parity of outputs the timed GPU run left behind."""
    threads = os.cpu_count() or 1
    cs = CpuSet(base, layers)
    cs.step(threads)  # warm
    times = []
    t_end = time.time() + seconds_target
    while time.time() < t_end and len(times) < 50:
        times.append(cs.step(threads))
    out = {"value": cs.nbytes / float(np.mean(times)) / 1e9, "unit": UNIT, "cores": threads, "kind": cs.kind,
           "sample": cs.describe(threads) + ", %d passes" % len(times)}
    # one thread: layer 0's seven matrices + lm_head
    idx = [i for i, (name, layer, n, k) in enumerate(cs.ops) if layer <= 0]
    nb1 = sum(shapes.mul_mat_bytes(cs.ops[i][2], cs.ops[i][3], 1) for i in idx)
    t0 = time.perf_counter()
    for i in idx:
        cs.run(cs.mats[i], cs.xs[cs.ops[i][3]], 1)
    out["one_thread"] = {"value": nb1 / (time.perf_counter() - t0) / 1e9, "unit": UNIT, "cores": 1,
                         "sample": "layer 0 q,k,v,o,gate,up,down + lm_head at M=1 (%.2f GB), one pass" % (nb1 / 1e9)}
    # prefill on the CPU: 512 tokens x 2048 rows of ffn_gate (a bounded slice of configs[3])
    rows = 2048
    wg = base["ffn_gate"][:rows]
    xp = synth.make_activation(512, shapes.E, 5)
    t0 = time.perf_counter()
    cs.run(wg, xp, threads)
    dt = time.perf_counter() - t0
    out["prefill_m512"] = {"value": shapes.mul_mat_flops(rows, shapes.E, 512) / dt / 1e9, "unit": "GFLOP/s", "cores": threads,
                           "sample": "512 tokens x %d rows of ffn_gate (K = 4096), Q8_0-quantised activations, one pass" % rows}
    parity = None
    if gpu_check is not None:
        from oracle import pyoracle as po

        orc = po.Oracle()
        parity = {"tolerance": 1e-4, "cases": {}}
        for label, w, x, y, rows_idx in gpu_check:
            ref = orc.mul_mat(po.Q8ACT_LANES, w if rows_idx is None else w[rows_idx], x)
            got = y if rows_idx is None else y[:, rows_idx]
            parity["cases"][label] = float(np.abs(got - ref).max() / np.abs(ref).max())
        parity["max_rel"] = max(parity["cases"].values())
        parity["ok"] = parity["max_rel"] <= 1e-4
    return out, parity


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    base, _ = host_weights()
    cs = CpuSet(base, args.layers)
    for _ in range(args.warmup):
        cs.step(threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cs.step(threads)
    sec = (time.perf_counter() - t0) / args.steps
    value = cs.nbytes / sec / 1e9
    weight_bytes = sum(n * (k // 32) * 34 for _, _, n, k in cs.ops)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": workload_config(args.layers, len(cs.ops), weight_bytes, "q8"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": cs.kind, "sample": cs.describe(threads)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(layers, n_ops, weight_bytes, act_mode):
    return {
        "workload": "configs[2]: LLaMA-3-8B full decode matmul set, batch 1: %d layers x (q,k,v,o,gate,up,down) + lm_head = %d Q8_0 mul_mats, "
                    "%.3f GB of Q8_0 weights per step" % (layers, n_ops, weight_bytes / 1e9),
        "act_mode": "q8_0 activations (reference quantiser), exact int8 block dots" if act_mode == "q8" else "f32 activations x dequantised weights",
    }


# ---------------------------------------------------------------------------------------------------------------
# GPU legs that ride along in the JSON line, outside the timed region
# ---------------------------------------------------------------------------------------------------------------
def prefill_run(ctx, stream, torch, ops, weights, base, timed, world, M=512, iters=10):
    """configs[3]: a 512-token activation matrix times layer 0's gate, up and down weights (this rank's row shards).
    Returns whole-job TFLOP/s (2*M*N*K flops per mul_mat), the fraction of the measured dense bf16 peak per GPU, and
    the parity inputs (outputs of the timed kernels) for the CPU checker."""
    by_name = {}
    for i, (name, layer, n, k) in enumerate(ops):
        if layer == 0 and name in ("ffn_gate", "ffn_up", "ffn_down"):
            by_name[name] = (weights[i], n, k)
    if len(by_name) != 3:
        return None, []
    out, checks = {}, []
    xh = {k: synth.make_activation(M, k, 777 + k) for k in {v[2] for v in by_name.values()}}
    with torch.cuda.stream(stream):
        xs = {k: torch.from_numpy(v).cuda() for k, v in xh.items()}
        ys = {name: torch.zeros((M, n), device="cuda") for name, (_, n, _) in by_name.items()}
    stream.synchronize()
    flops_total, ms_sum = 0, 0.0
    for name, (w, n, k) in by_name.items():
        fn = lambda: ctx.mul_mat(w, xs[k], ys[name])  # noqa: E731
        for _ in range(3):
            fn()
        ctx.sync()
        ms = timed(fn, iters) / iters
        plan = ctx.capi.gemm_tile_plan(w.n1 - w.n0, M)
        out[name] = {"N": n, "K": k, "M": M, "ms": ms, "tflops": shapes.mul_mat_flops(n, k, M) / (ms * 1e-3) / 1e12,
                     "tile": "%s x %d" % ("tokens on lanes" if plan["swapped"] else "rows on lanes", plan["tile_cols"])}
        flops_total += shapes.mul_mat_flops(n, k, M)
        ms_sum += ms
        # this rank's rows of the output the timed kernel wrote, a strided subset of them for the CPU checker
        idx = np.arange(w.n0, w.n1, 37)
        checks.append(("prefill_%s_m%d" % (name, M), base[name], xh[k], ys[name].cpu().numpy(), idx))
    _, tf_peak, kind = measured_peaks()
    agg = flops_total / (ms_sum * 1e-3) / 1e12
    return ({"workload": "configs[3]: M=512 x (gate, up 14336x4096; down 4096x14336), Q8_0 weights, Q8_0-quantised activations",
             "tflops": agg, "per_gpu_tflops": agg / world, "frac_of_bf16_peak": agg / world / tf_peak, "peak_tflops": tf_peak, "peak_kind": kind,
             "per_op": out, "note": "outside the timed decode region; weights of one layer (187 MB) exceed L2"}, checks)


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


def noalloc_run(ctx, stream, torch, ops, weights, timed, iters=20):
    """The allocation-free entry point (nhb_mul_mat_q8_0_noalloc) on the attn_q weights of up to 8 layers, M = 1: per call
    one quantise launch + one GEMV launch from raw plane pointers."""
    capi = ctx.capi
    ws = [(weights[i], n, k) for i, (name, layer, n, k) in enumerate(ops) if name == "attn_q" and weights[i].n1 - weights[i].n0 == n][:8]
    if not ws:
        return None
    with torch.cuda.stream(stream):
        x = torch.randn((1, ws[0][2]), device="cuda")
        ys = [torch.zeros((1, n), device="cuda") for _, n, _ in ws]

    def run():
        for (w, n, k), y in zip(ws, ys):
            rc = capi.lib.nhb_mul_mat_q8_0_noalloc(w.q_ptr, w.d_ptr, n, k, x.data_ptr(), k, y.data_ptr(), n, 1, stream.cuda_stream)
            if rc != 0:
                raise RuntimeError(capi.lib.nhb_noalloc_last_error().decode())

    run()
    stream.synchronize()
    ms = timed(run, iters) / iters
    nbytes = sum(shapes.mul_mat_bytes(n, k, 1) for _, n, k in ws)
    return {"workload": "attn_q 4096x4096, M=1, %d layers in rotation (%.0f MB), host-issued calls (no graph)" % (len(ws), nbytes / 1e6),
            "us_per_call": ms * 1e3 / len(ws), "gbs": nbytes / (ms * 1e-3) / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=shapes.L, help="debug: fewer layers (the reported workload is 32)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--act-mode", default="q8", choices=["q8", "f32"],
                    help="q8: activations quantised to Q8_0, exact int8 block dots (the reported metric); f32: f32 activations x dequantised weights")
    ap.add_argument("--replicate-mb", type=int, default=48,
                    help="N > 1 placement policy: weights smaller than this many MiB stay whole on every rank (no exchange); 0 shards all")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl", "none"],
                    help="N > 1: outputs completed by the GEMV's own peer stores (fused) or by a grouped NCCL all-gather per stage")
    ap.add_argument("--peer-window", type=int, default=4,
                    help="N > 1, fused gather: a launch waits for the other ranks only if it reads rows they deliver, or to stay within this "
                         "many delivering launches of the slowest rank; 0 = every launch waits for every earlier delivery")
    ap.add_argument("--stage-times", action="store_true",
                    help="also time each stage type on its own (graphs of one launch per layer) and add `stage_us` to the JSON line")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 512-token GEMM, the rms_norm and the no-alloc figures that ride along in the JSON line")
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
    ctx.capi = capi
    if world > 1:
        ctx.set_option("replicate_below_mb", args.replicate_mb)
        ctx.set_option("peer_window", args.peer_window)
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
        weights.append(ctx.upload(layer_weight(base, name, layer)))
    upload_s = time.time() - t0
    # stages: (q,k,v) (o) (gate,up) (down) per layer, then lm_head; the ops of a stage read ONE input vector
    stages, i = [], 0
    for layer in range(args.layers):
        for stage in shapes.LAYER_STAGES:
            stages.append(list(range(i, i + len(stage))))
            i += len(stage)
    stages.append([i])
    x_off, y_off = [], []
    xo = yo = 0
    for st in stages:
        x_off.append(xo)
        xo += ops[st[0]][3]
    for name, layer, n, k in ops:
        y_off.append(yo)
        yo += n
    x_host = torch.empty(xo, dtype=torch.float32).pin_memory()
    rng = np.random.default_rng(synth.seed_for(2, "attn_q", "activations"))
    x_host.numpy()[:] = rng.standard_normal(xo, dtype=np.float32)
    y_host = torch.empty(yo, dtype=torch.float32).pin_memory()
    fused = world > 1 and args.gather == "fused"
    with torch.cuda.stream(stream):
        x_dev = x_host.to("cuda", non_blocking=True)
        # with several ranks the outputs live in symmetric memory and the GEMV delivers every rank's columns itself
        y_dev = ctx.symm_empty((yo,)) if fused else torch.zeros(yo, dtype=torch.float32, device="cuda")
    stream.synchronize()
    xs = [x_dev[x_off[s]:x_off[s] + ops[st[0]][3]].view(1, -1) for s, st in enumerate(stages)]
    ys = [y_dev[y_off[j]:y_off[j] + ops[j][2]].view(1, -1) for j in range(len(ops))]
    act_mode = capi.ACT_Q8 if args.act_mode == "q8" else capi.ACT_F32

    # A stage chain records the whole step once (Q8 arithmetic).  A stage's rows are whole on every rank before the next
    # stage reads its input: with fused delivery every launch waits for the peers' announcements in its prologue and the
    # step ends with one explicit wait for the last stage; with NCCL every stage is followed by its grouped all-gather.
    chain = None
    if act_mode == capi.ACT_Q8 and (world == 1 or fused):
        chain = ctx.chain([[(weights[j], xs[s], ys[j]) for j in st] for s, st in enumerate(stages)])

    def enqueue_step():
        if chain is not None:
            chain.launch()
            if world > 1:
                ctx.all_gather_batch([ys[j] for j in stages[-1]])
            return
        for s, st in enumerate(stages):
            ctx.mul_mat_batch([(weights[j], xs[s], ys[j]) for j in st], act_mode=act_mode)
            if world > 1 and args.gather != "none":  # "none" leaves the rows incomplete: timing experiments only
                ctx.all_gather_batch([ys[j] for j in st])

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

    def timed(fn, steps, stamps=None):
        ev0 = torch.cuda.Event(enable_timing=True)
        ev1 = torch.cuda.Event(enable_timing=True)
        barrier()
        t_begin = time.perf_counter()
        with torch.cuda.stream(stream):
            ev0.record(stream)
            for _ in range(steps):
                fn()
            ev1.record(stream)
        ctx.sync()
        t_end = time.perf_counter()
        barrier()
        if stamps is not None:
            stamps.extend([t_begin, t_end])
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step()
    ctx.sync()
    stamps = []
    ms_total = timed(step, args.steps, stamps)
    clocks = sampler.window(stamps[0], stamps[1])
    ms_step = ms_total / args.steps

    # ---- end to end: host activations in, host outputs out, through the C ABI every step ----
    x_bytes, y_bytes = xo * 4, yo * 4

    def e2e_step():
        # every rank needs the step's inputs; the complete outputs (the same on every rank) go back to the host once, from rank 0
        ctx.memcpy_h2d(x_dev.data_ptr(), x_host.data_ptr(), x_bytes)
        step()
        if rank == 0:
            ctx.memcpy_d2h(y_host.data_ptr(), y_dev.data_ptr(), y_bytes)

    for _ in range(3):
        e2e_step()
    ctx.sync()
    e2e_steps = max(10, args.steps // 4)
    e2e_ms = timed(e2e_step, e2e_steps) / e2e_steps
    sampler.stop()
    if rank != 0:  # untimed: the parity check below compares every rank's buffer
        ctx.memcpy_d2h(y_host.data_ptr(), y_dev.data_ptr(), y_bytes)
        ctx.sync()
    y_after = y_host.numpy().copy()  # the outputs of the last end-to-end step, as the host received them

    # ---- the same step with every launch waiting for every earlier delivery (what a step costs when each stage reads the
    #      rows the stage before it gathered); the stages of the timed workload read independent synthetic vectors ----
    lockstep_ms = None
    if fused and graph is not None and args.peer_window != 0:
        ctx.set_option("peer_window", 0)
        ctx.graph_begin()
        enqueue_step()
        g0 = ctx.graph_end()
        for _ in range(5):
            g0.launch()
        ctx.sync()
        n0 = max(20, args.steps // 4)
        lockstep_ms = timed(g0.launch, n0) / n0
        g0.free()
        ctx.set_option("peer_window", args.peer_window)

    # ---- the step as the data flow of a decode step: every stage reads what the stage before it wrote (down -> q,k,v;
    #      q -> attn_output; attn_output -> gate,up; gate -> down; the last down -> lm_head), so with N > 1 a stage waits for
    #      the ranks that deliver its input.  Attention, SwiGLU, norms and residuals are left out: only the dependency is modelled ----
    dependent_ms = None
    if chain is not None and graph is not None:
        dep_in, prev = [], None
        for s, st in enumerate(stages):
            names = [ops[j][0] for j in st]
            if prev is None:
                dep_in.append(xs[s])
            elif names[0] in ("attn_q", "output"):
                dep_in.append(ys[prev["down"]])
            elif names[0] == "attn_output":
                dep_in.append(ys[prev["q"]])
            elif names[0] == "ffn_gate":
                dep_in.append(ys[prev["o"]])
            else:
                dep_in.append(ys[prev["gate"]])
            prev = dict(prev or {})
            prev[{"attn_q": "q", "attn_output": "o", "ffn_gate": "gate", "ffn_down": "down"}.get(names[0], "x")] = st[0]
        dchain = ctx.chain([[(weights[j], dep_in[s], ys[j]) for j in st] for s, st in enumerate(stages)])

        def enqueue_dependent():
            dchain.launch()
            if world > 1:
                ctx.all_gather_batch([ys[j] for j in stages[-1]])

        enqueue_dependent()
        ctx.sync()
        ctx.graph_begin()
        enqueue_dependent()
        gd = ctx.graph_end()
        for _ in range(5):
            gd.launch()
        ctx.sync()
        nd = max(20, args.steps // 4)
        dependent_ms = timed(gd.launch, nd) / nd
        gd.free()
        dchain.free()

    # ---- each stage type on its own: one launch per layer, recorded and replayed like the step ----
    stage_us = None
    if args.stage_times and act_mode == capi.ACT_Q8 and args.gather != "nccl":
        stage_us = {}
        per_layer = len(shapes.LAYER_STAGES)
        peak_gbs = measured_peaks()[0]
        for t, label in enumerate("+".join(n.replace("attn_", "").replace("ffn_", "") for n in st) for st in shapes.LAYER_STAGES):
            idx = [per_layer * layer + t for layer in range(args.layers)]
            ch = ctx.chain([[(weights[j], xs[s], ys[j]) for j in stages[s]] for s in idx])

            def enqueue_stage(ch=ch, last=stages[idx[-1]]):
                ch.launch()
                if fused:
                    ctx.all_gather_batch([ys[j] for j in last])

            enqueue_stage()
            ctx.sync()
            ctx.graph_begin()
            enqueue_stage()
            g = ctx.graph_end()
            for _ in range(5):
                g.launch()
            ctx.sync()
            reps = 50
            us = timed(g.launch, reps) / reps * 1e3 / len(idx)
            g.free()
            ch.free()
            nb = sum(weights[j].bytes_q8 + 4 * ops[j][3] + 4 * (weights[j].n1 - weights[j].n0) for j in stages[idx[0]])
            stage_us[label] = {"us_per_launch": us, "rank_mb": nb / 1e6, "bytes_over_peak_us": nb / peak_gbs / 1e3,
                               "delivers": bool(fused and any(weights[j].n1 - weights[j].n0 < ops[j][2] for j in stages[idx[0]]))}

    total_bytes = sum(shapes.mul_mat_bytes(n, k, 1) for _, _, n, k in ops)
    weight_bytes = sum(n * (k // 32) * 34 for _, _, n, k in ops)
    value = total_bytes / (ms_step * 1e-3) / 1e9
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e9
    hbm_peak, _, peak_kind = measured_peaks()
    # what THIS rank streams per step under the placement policy: its row shard of every weight, whole or split
    rank_weight_bytes = sum(w.bytes_q8 for w in weights)
    rank_bytes = rank_weight_bytes + sum(4 * k + 4 * (w.n1 - w.n0) for (_, _, n, k), w in zip(ops, weights))

    # ---- parity of the timed buffers ----
    # every rank must hold the same complete outputs (delivered rows included) ...
    digest = int(torch.from_numpy(y_after.view(np.int32)).to(torch.int64).sum().item()) & 0xFFFFFFFFFFFF
    all_equal = True
    if world > 1:
        t = torch.tensor([digest], dtype=torch.int64, device="cuda")
        gathered = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        all_equal = all(int(g.item()) == digest for g in gathered)
    # ... and they are checked against the CPU oracle in the CPU leg below (1 GPU), or against an unsharded
    # single-context run of the same stages on this GPU (N > 1: "the same numbers as one GPU")
    gpu_check = []
    for label, j in (("layer0_ffn_gate", next(j for j, o in enumerate(ops) if o[0] == "ffn_gate")),
                     ("layer0_ffn_down", next(j for j, o in enumerate(ops) if o[0] == "ffn_down")), ("lm_head", len(ops) - 1)):
        s = next(s for s, st in enumerate(stages) if j in st)
        xh = x_host.numpy()[x_off[s]:x_off[s] + ops[j][3]][None, :]
        yh = y_after[y_off[j]:y_off[j] + ops[j][2]][None, :]
        idx = None if ops[j][2] <= 16384 else np.arange(0, ops[j][2], 13)
        gpu_check.append((label, layer_weight(base, ops[j][0], ops[j][1]), xh, yh, idx))
    one_gpu_equal = None
    if world > 1 and rank == 0:
        solo = capi.Context(local, 0, 1)
        solo.set_stream(stream.cuda_stream)
        one_gpu_equal = True
        for label, w, xh, yh, idx in gpu_check[:2]:
            h = solo.upload(w)
            with torch.cuda.stream(stream):
                got = solo.mul_mat(h, torch.from_numpy(np.ascontiguousarray(xh)).cuda())
            solo.sync()
            one_gpu_equal = one_gpu_equal and bool((got.cpu().numpy().view(np.uint32) == yh.view(np.uint32)).all())
            h.free()
        solo.close()

    # ---- prefill (configs[3]), rms_norm and the allocation-free entry point: outside the timed region ----
    prefill, norm, noalloc = None, None, None
    if not args.no_prefill:
        prefill, pchecks = prefill_run(ctx, stream, torch, ops, weights, base, timed, world)
        gpu_check.extend(pchecks)
        if world == 1 and args.act_mode == "q8":
            norm = norm_run(ctx, stream, torch, ops, weights, timed)
            noalloc = noalloc_run(ctx, stream, torch, ops, weights, timed)

    if rank == 0:
        n_launch = len(stages)
        per_launch_bytes = rank_bytes / n_launch
        per_launch_ms = ms_step / n_launch
        per_gpu_gbs = rank_bytes / (ms_step * 1e-3) / 1e9
        config = workload_config(args.layers, len(ops), weight_bytes, args.act_mode)
        config.update({
            "launch_grouping": "one launch per stage (the independent projections of a stage together), recorded as a stage chain" if chain is not None else "one launch per stage",
            "cuda_graph": graph is not None,
            "parallelism": "row-shard x%d" % world + ("" if world == 1 or not args.replicate_mb else " (weights under %d MiB replicated)" % args.replicate_mb) +
                           ("" if world == 1 else (" + all-gather fused into the GEMV (peer stores over NVLink; a launch waits for the peers when it reads delivered rows, "
                                                   "the step ends with a wait for every delivery; window %d)" % args.peer_window if fused else " + NCCL all-gather per stage")),
            "l2": "inputs larger than L2 (this rank streams %.2f GB of weights per step vs 126 MB)" % (rank_weight_bytes / 1e9),
        })
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic", "config": config,
            "tokens_per_s_equiv": 1e3 / ms_step,
            "frac_of_nominal_8TBs": per_gpu_gbs / NOMINAL_HBM_GBS,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_bytes, "d2h_bytes_per_step": y_bytes, "ms_per_step": e2e_ms},
            "gpu_launches": launches_per_step * args.steps,
            "launches_per_step": launches_per_step,
            "clocks": clocks,
            "ms_per_step_x_sm_mhz": (ms_step * clocks["sm_mhz"]) if clocks.get("sm_mhz") else None,
            "roofline": {
                "bound": "hbm", "kernel": "gemv_q8_rows", "achieved": per_launch_bytes / (per_launch_ms * 1e-3) / 1e9, "peak": hbm_peak,
                "unit": "GB/s", "frac": per_launch_bytes / (per_launch_ms * 1e-3) / 1e9 / hbm_peak, "peak_kind": peak_kind,
                "traffic": (NCU_DRAM_BYTES_PER_STEP / n_launch) if (args.layers == shapes.L and world == 1) else None,
                "bytes_per_launch": per_launch_bytes, "ms_per_launch": per_launch_ms,
                "note": "per GPU: the bytes this rank streams under the placement policy; launch gaps inside the graph are included in the duration",
            },
            "every_launch_waits_ms_per_step": lockstep_ms,
            "dependent_chain_ms_per_step": dependent_ms,
            "stage_us": stage_us,
            "parity": {"all_ranks_hold_the_same_outputs": all_equal, "bit_identical_to_one_gpu": one_gpu_equal},
            "prefill": prefill,
            "rms_norm": norm,
            "noalloc": noalloc,
            "setup_s": {"generate": gen_s, "upload": upload_s},
        }
        if world == 1 and not args.no_cpu_baseline:
            cpu, parity = cpu_baseline_leg(base, args.layers, args.cpu_seconds, gpu_check)
            line["cpu_baseline"] = cpu
            line["parity"].update(parity)
            if prefill is not None:
                prefill["parity_max_rel"] = max(v for k, v in parity["cases"].items() if k.startswith("prefill_"))
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)

    if graph is not None:
        graph.free()
    if chain is not None:
        chain.free()
    for w in weights:
        w.free()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
