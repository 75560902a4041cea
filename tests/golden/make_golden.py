"""Generates tests/golden/q8_ref_vectors.npz from the reference's own helpers.

Run in a container that has the reference tree (it builds oracle/_ref/libnihilus_ref.so from the
reference's cpu/avx_2.hpp in place, see oracle/build_ref.sh):

    python tests/golden/make_golden.py

The fixture holds seeded inputs and the outputs of the reference functions
quantize_row_q8_0 (cpu/avx_2.hpp:4439-4489), vec_dot_q8_0_q8_0_impl (:4749-4780), the <=16-block
vec_dot_q8_0_q8_0<n> kernels chained as the >16 driver does (:4536-4747), vec_dot_q8_f32<K>
(:4800-4852), scalar_dot_product_q8_f32 (:4881-4907) and the fp16 converters (cpu/common.hpp:215-221),
so the oracle can be pinned on machines where the reference tree is absent.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import pyoracle  # noqa: E402

SHAPES = [(8, 32), (8, 64), (8, 96), (6, 128), (6, 512), (5, 1024), (4, 4096), (3, 14336)]  # (rows, K)


def main() -> None:
    pyoracle.build()
    ref = pyoracle.Reference()
    rng = np.random.default_rng(20250101)
    out = {}
    # fp16 conversion samples: all interesting magnitudes + every half code
    f = np.concatenate([rng.standard_normal(4096).astype(np.float32) * s for s in (1e-8, 6e-8, 1e-5, 6.1e-5, 1e-3, 1.0, 1e3, 65504.0, 7e4)])
    f = np.concatenate([f, np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 5.9604645e-8, 2.9802322e-8, 2.98023224e-8 * 1.0000001, np.inf, -np.inf],
                                    dtype=np.float32)])
    out["fp16_in"] = f
    out["fp16_out"] = np.array([ref.fp32_to_fp16(float(v)) for v in f], dtype=np.uint16)
    out["fp16_bittrick_out"] = np.array([ref.fp32_to_fp16_bittrick(float(v)) for v in f], dtype=np.uint16)
    out["fp16_codes_to_f32"] = np.array([ref.fp16_to_fp32(h) for h in range(65536)], dtype=np.float32).view(np.uint32)
    for i, (rows, K) in enumerate(SHAPES):
        w = (rng.standard_normal((rows, K)) * 0.02).astype(np.float32)
        x = rng.standard_normal((2, K)).astype(np.float32)
        if i == 0:  # known-answer style rows: zero block, saturating block, single spike, tiny scale
            x[0, :32] = 0.0
            x[1, :32] = 0.0
            x[1, 7] = 3.0
            w[0, :32] = 0.0
            w[1, :32] = np.where(np.arange(32) % 2 == 0, 1.0, -1.0)
            w[2, :32] = 0.0
            w[2, 31] = -5.0
            w[3, :32] = (rng.standard_normal(32) * 1e-7).astype(np.float32)
        wq = ref.quantize_rows(w)
        aq = ref.quantize_rows(x)
        out[f"w_f32_{i}"] = w
        out[f"x_f32_{i}"] = x
        out[f"w_blocks_{i}"] = wq
        out[f"x_blocks_{i}"] = aq
        out[f"dot_lanes_{i}"] = np.array([[ref.vec_dot_q8q8(wq[n], aq[m]) for n in range(rows)] for m in range(2)], dtype=np.float32)
        out[f"dot_chunk16_{i}"] = np.array([[ref.vec_dot_q8q8(wq[n], aq[m], chunk16=True) for n in range(rows)] for m in range(2)],
                                           dtype=np.float32)
        out[f"dot_f32_eval_{i}"] = np.array([[ref.vec_dot_q8f32(wq[n], x[m]) for n in range(rows)] for m in range(2)], dtype=np.float32)
        out[f"dot_f32_prompt_{i}"] = np.array([[ref.vec_dot_q8f32(wq[n], x[m], prompt=True) for n in range(rows)] for m in range(2)],
                                              dtype=np.float32)
    out["shapes"] = np.array(SHAPES, dtype=np.int64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "q8_ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
