"""Seeded synthetic inputs with the shapes and distributions of the LLaMA-3-8B Q8_0 workload.

Weights are f32 ~ N(0, 0.02^2) quantised to Q8_0 along K exactly like the reference's quantiser
(include/nihilus-incl/cpu/avx_2.hpp:4439-4489): per 32 values d = fp16(amax / 127), q = rint(x * (127 / amax)).
Activations are f32 ~ N(0, 1).  numpy's float32 arithmetic is IEEE, so the blocks produced here are
byte-identical to the CPU oracle's (checked in the tests); this module does not depend on the oracle.
"""
from __future__ import annotations

import numpy as np

TENSOR_IDS = {"attn_q": 0, "attn_k": 1, "attn_v": 2, "attn_output": 3, "ffn_gate": 4, "ffn_up": 5, "ffn_down": 6, "output": 7}


def seed_for(config: int, tensor: str, kind: str, layer: int = 0) -> int:
    """20250000 + 1000*config + 100*layer*... : one stream per (config, tensor, weights|activations, layer)."""
    return 20250000 + 1000 * config + 10 * TENSOR_IDS[tensor] + (0 if kind == "weights" else 1) + 100000 * max(layer, 0)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """f32 [rows, K] -> uint8 [rows, K/32, 34] Q8_0 blocks {fp16 d (little endian); int8 qs[32]}."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, K = x.shape
    assert K % 32 == 0
    xb = x.reshape(rows, K // 32, 32)
    amax = np.abs(xb).max(axis=2)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(amax != 0, np.float32(127.0) / amax, np.float32(0.0)).astype(np.float32)
    q = np.rint(xb * inv[:, :, None]).clip(-128, 127).astype(np.int8)
    out = np.empty((rows, K // 32, 34), dtype=np.uint8)
    out[:, :, 0:2] = d.astype(np.float16).view(np.uint8).reshape(rows, K // 32, 2)
    out[:, :, 2:] = q.view(np.uint8)
    return out


def make_weight(N: int, K: int, seed: int, chunk_rows: int = 2048, threads: int | None = None) -> np.ndarray:
    """Q8_0 blocks of an [N, K] weight drawn from N(0, 0.02^2).

    Row chunks are drawn from independent child streams of `seed` (SeedSequence.spawn), so the result does
    not depend on the number of worker threads.
    """
    import os
    from concurrent.futures import ThreadPoolExecutor

    out = np.empty((N, K // 32, 34), dtype=np.uint8)
    starts = list(range(0, N, chunk_rows))
    children = np.random.SeedSequence(seed).spawn(len(starts))

    def work(i: int) -> None:
        r0 = starts[i]
        r1 = min(N, r0 + chunk_rows)
        rng = np.random.default_rng(children[i])
        w = rng.standard_normal((r1 - r0, K), dtype=np.float32)
        w *= np.float32(0.02)
        out[r0:r1] = quantize_q8_0(w)

    threads = threads or min(32, os.cpu_count() or 1)
    if threads <= 1 or len(starts) == 1:
        for i in range(len(starts)):
            work(i)
    else:
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(work, range(len(starts))))
    return out


def make_activation(M: int, K: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((M, K), dtype=np.float32)


def roll_rows(blocks: np.ndarray, shift: int) -> np.ndarray:
    """A distinct weight of the same distribution for another layer: the same rows, rotated."""
    return np.roll(blocks, shift, axis=0)
