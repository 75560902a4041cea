"""Generates tests/golden/rms_norm_ref_vectors.npz from the reference's own helpers.

Run in a container that has the reference tree (oracle/build_ref.sh compiles the reference's
simd_sum_squares, sqrtf_fast, vec_scale_mul_f32<K> and quantize_row_q8_0_avx2 in place):

    python tests/golden/make_golden_rms_norm.py

The fixture holds seeded rows, norm weights and, for both sqrtf_fast builds (0 = IEEE root, 1 = the x86 integer
formula), the f32 rows and the Q8_0 blocks those reference functions produce (cpu/avx_2.hpp:671-779, 3621-3850,
3907-3915; cpu/common.hpp:448-450), so the oracle can be pinned where the reference tree is absent.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import pyoracle  # noqa: E402

SHAPES = [(4, 32), (3, 96), (3, 160), (2, 512), (2, 4096), (1, 14336)]  # (rows, K): every K is instantiated in ref_postlude.cpp
EPS = (1e-5, 1e-6)


def main() -> None:
    pyoracle.build()
    ref = pyoracle.Reference()
    rng = np.random.default_rng(20250607)
    out = {"eps": np.array(EPS, dtype=np.float32)}
    for i, (rows, K) in enumerate(SHAPES):
        x = (rng.standard_normal((rows, K)) * rng.uniform(0.05, 20.0, (rows, 1))).astype(np.float32)
        x[0, : min(K, 32)] = 0.0  # one all-zero Q8 block
        w = rng.uniform(0.1, 2.5, K).astype(np.float32)
        out[f"x{i}"], out[f"w{i}"] = x, w
        out[f"sumsq{i}"] = np.array([ref.sum_squares(r) for r in x], dtype=np.float32).view(np.uint32)
        for mode in (0, 1):
            for e, eps in enumerate(EPS if K < 4096 else EPS[:1]):  # the long rows once, to keep the fixture small
                out[f"y{i}_m{mode}_e{e}"] = ref.rms_norm_mul(x, w, float(np.float32(eps)), mode).view(np.uint32)
                out[f"q{i}_m{mode}_e{e}"] = ref.rms_norm_mul_q8_0(x, w, float(np.float32(eps)), mode)
    v = np.concatenate([rng.uniform(1e-8, 4.0, 256), rng.uniform(4.0, 1e6, 256)]).astype(np.float32)
    out["sqrt_in"] = v
    out["sqrt_fast_out"] = np.array([ref.sqrtf_fast(float(t)) for t in v], dtype=np.float32).view(np.uint32)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rms_norm_ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
