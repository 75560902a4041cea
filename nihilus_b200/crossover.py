"""Crossover sweep: times the decode GEMV and the tensor-core GEMM for a range of token counts M on the LLaMA-3-8B
projection shapes and reports where the GEMM starts to win (the value `gemv_max_m` should have on this GPU).

    python -m nihilus_b200.crossover [--ms 1 2 4 8 16 32 64 128 2048] [--shapes attn_q ffn_gate ...] [--world G]

Prints one JSON line per (shape, M) with both kernels' time, GB/s and TFLOP/s, then one summary line per shape.
`--world G` times the row shard one of G GPUs would own (rows / G) on this GPU.  Weights are synthetic Q8_0 blocks
(a 2048-row pattern repeated: values do not matter for timing); every timing rotates over enough distinct weight
copies to exceed the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def _time(fn, stream, torch, reps: int) -> float:
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(3):
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        stream.synchronize()
        best = min(best, e0.elapsed_time(e1) / reps)
    return best  # ms per pass


def main() -> None:
    import torch

    from . import capi, shapes, synth

    ap = argparse.ArgumentParser()
    ap.add_argument("--ms", type=int, nargs="*", default=[1, 2, 4, 8, 16, 32, 64, 128, 2048])
    ap.add_argument("--shapes", nargs="*", default=["attn_q", "attn_k", "attn_output", "ffn_gate", "ffn_down", "output"])
    ap.add_argument("--world", type=int, default=1)
    args = ap.parse_args()

    ctx = capi.Context(0)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    pattern = {}
    for name in args.shapes:
        n_full, k = shapes.LLAMA3_8B[name]
        n = max(1, n_full // args.world)
        if k not in pattern:
            pattern[k] = synth.make_weight(2048, k, 7)
        base = np.concatenate([pattern[k]] * (n // 2048 + 1))[:n]
        copies = max(2, int(np.ceil(400e6 / (n * (k // 32) * 34))))  # > 3x L2 in rotation
        copies = min(copies, 24)
        ws = [ctx.upload(np.roll(base, 3 * i, axis=0)) for i in range(copies)]
        switch = None
        for m in args.ms:
            with torch.cuda.stream(stream):
                x = torch.randn((m, k), device="cuda")
                y = torch.zeros((m, n), device="cuda")
            row = {"shape": name, "N": n, "K": k, "M": m, "world": args.world}
            for label, kern in (("gemv", capi.KERNEL_GEMV_ROWS), ("gemm", capi.KERNEL_GEMM_TC)):
                if label == "gemv" and m > 128:
                    continue  # M / 4 passes over the weights: never competitive, and slow to time

                def run(kern=kern):
                    for w in ws:
                        ctx.mul_mat(w, x, y, kernel=kern)

                run()
                ctx.sync()
                ms = _time(run, stream, torch, 2) / copies
                row[label + "_us"] = round(ms * 1e3, 2)
                row[label + "_gbs"] = round(shapes.mul_mat_bytes(n, k, m) / ms / 1e6, 1)
                row[label + "_tflops"] = round(shapes.mul_mat_flops(n, k, m) / ms / 1e9, 2)
            if switch is None and "gemv_us" in row and row["gemm_us"] < row["gemv_us"]:
                switch = m
            print(json.dumps(row), flush=True)
        print(json.dumps({"shape": name, "N": n, "K": k, "world": args.world, "gemm_wins_from_M": switch}), flush=True)
        for w in ws:
            w.free()
    ctx.close()


if __name__ == "__main__":
    main()
