"""The C-ABI library: loads without a GPU, exports what the header declares, host-side logic (no GPU compute)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "nihilus_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nhb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(capi):
    declared = _declared_symbols()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(capi.lib, name), f"{name} declared in include/nihilus_b200.h but not exported"
    assert sorted(capi.EXPORTS) == declared


def test_version_and_arch(capi):
    assert capi.lib.nhb_version() == 100
    assert capi.lib.nhb_arch() == 100


def test_shard_rows(capi):
    for N in (0, 1, 7, 1024, 4096, 14336, 128256):
        for world in (1, 2, 3, 4, 8):
            prev = 0
            sizes = []
            for r in range(world):
                a, b = capi.shard_rows(N, world, r)
                assert a == prev and b >= a
                prev = b
                sizes.append(b - a)
            assert prev == N and max(sizes) - min(sizes) <= 1
    with pytest.raises(capi.NhbError):
        capi.shard_rows(10, 2, 2)
    with pytest.raises(capi.NhbError):
        capi.shard_rows(-1, 1, 0)


def test_repack_host_round_trip_and_matches_oracle(capi, oracle):
    rng = np.random.default_rng(4)
    w = oracle.quantize_rows((rng.standard_normal((21, 160)) * 0.02).astype(np.float32))
    for n0, n1 in ((0, 21), (5, 13), (7, 7)):
        q, d = capi.repack_host(w, n0, n1)
        qo, do = oracle.repack(w, n0, n1)
        assert (q == qo).all() and (d == do).all()
        assert (capi.unpack_host(q, d) == w[n0:n1]).all()
    with pytest.raises(capi.NhbError):
        capi.lib.nhb_repack_q8_0_host.restype = C.c_int
        capi._check(capi.lib.nhb_repack_q8_0_host(w.ctypes.data, 21, 100, 0, 21, w.ctypes.data, w.ctypes.data))  # K % 32 != 0


def test_choose_kernel_and_work_formulas(capi):
    from nihilus_b200 import shapes

    assert capi.lib.nhb_choose_kernel(4096, 4096, 1, capi.ACT_Q8) == capi.KERNEL_GEMV_ROWS
    assert capi.lib.nhb_choose_kernel(4096, 4096, 8, capi.ACT_Q8) == capi.KERNEL_GEMV_ROWS
    assert capi.lib.nhb_choose_kernel(4096, 96, 1, capi.ACT_Q8) == capi.KERNEL_GEMV_ROWS
    assert capi.lib.nhb_choose_kernel(4096, 4096, 512, capi.ACT_Q8) == capi.KERNEL_GEMM_TC
    assert capi.lib.nhb_choose_kernel(4096, 4096, 1, capi.ACT_F32) == capi.KERNEL_GEMV_ROWS
    assert capi.lib.nhb_choose_kernel(4096, 65536, 1, capi.ACT_F32) == capi.KERNEL_GEMV_LDG
    assert capi.lib.nhb_mul_mat_bytes(4096, 4096, 1) == 17825792 + 16384 + 16384 == shapes.mul_mat_bytes(4096, 4096, 1)
    assert capi.lib.nhb_mul_mat_flops(14336, 4096, 512) == 2 * 512 * 14336 * 4096 == shapes.mul_mat_flops(14336, 4096, 512)
    total = sum(n * (k // 32) * 34 for _, _, n, k in shapes.decode_set())
    assert total == 7973699584 and len(shapes.decode_set()) == 225


def test_no_gpu_means_loud_failure_not_fallback(capi):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = capi.lib.nhb_ctx_create(C.byref(h), 0, 0, 1)
    assert rc == capi.ERR_CUDA and not h.value
    assert "cuda" in capi.last_error().lower()
    with pytest.raises(capi.NhbError):
        capi.Context(0)


def test_bad_context_arguments(capi):
    h = C.c_void_p()
    assert capi.lib.nhb_ctx_create(C.byref(h), 0, 3, 2) == capi.ERR_ARG
    assert capi.lib.nhb_ctx_create(None, 0, 0, 1) == capi.ERR_ARG
    assert capi.lib.nhb_sync(None) == capi.ERR_ARG
    assert capi.lib.nhb_ctx_destroy(None) == capi.OK
    assert capi.lib.nhb_weight_free(None, None) == capi.OK


def test_product_does_not_touch_the_oracle():
    """No file of the package or the library sources may import, include or load anything under oracle/."""
    pkg = os.path.join(ROOT, "nihilus_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(base, f), errors="ignore").read()
                assert "pyoracle" not in text and "q8_oracle" not in text and "liboracle" not in text, os.path.join(base, f)
    for f in os.listdir(os.path.join(ROOT, "include")):
        p = os.path.join(ROOT, "include", f)
        if os.path.isfile(p):
            assert "oracle" not in open(p).read()


def test_placement_policy_replicates_small_weights_only(capi):
    """LLaMA-3-8B at 8 ranks with a 48 MiB threshold: q, k, v, attn_output whole on every rank, the FFN and lm_head sharded."""
    from nihilus_b200 import shapes

    thr = 48 << 20
    for name, (n, k) in shapes.LLAMA3_8B.items():
        covered = []
        for r in range(8):
            n0, n1 = capi.place_rows(n, k, 8, r, thr)
            if name in ("attn_q", "attn_k", "attn_v", "attn_output"):
                assert (n0, n1) == (0, n)
            else:
                assert (n0, n1) == capi.shard_rows(n, 8, r)
                covered.append((n0, n1))
        if covered:
            assert covered[0][0] == 0 and covered[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
        assert capi.place_rows(n, k, 1, 0, thr) == (0, n)  # one rank: nothing to decide
        assert capi.place_rows(n, k, 8, 3, 0) == capi.shard_rows(n, 8, 3)  # policy off


def test_gemm_tile_plan_covers_the_output_and_fills_waves(capi):
    for rows in (1, 100, 1024, 4096, 14336, 128256):
        for M in (9, 16, 64, 127, 128, 130, 512, 2048):
            p = capi.gemm_tile_plan(rows, M)
            lanes, cols = (M, rows) if p["swapped"] else (rows, M)
            assert p["tile_cols"] % 16 == 0 and 16 <= p["tile_cols"] <= 256
            assert p["lane_tiles"] * 128 >= lanes and (p["lane_tiles"] - 1) * 128 < lanes
            assert p["col_tiles"] * p["tile_cols"] >= cols and (p["col_tiles"] - 1) * p["tile_cols"] < cols
    # few tokens: weight rows on the lanes, the tokens (rounded up to 16) on the columns
    p = capi.gemm_tile_plan(14336, 16)
    assert not p["swapped"] and p["tile_cols"] == 16
    # the configs of the prefill benchmark: tokens on the lanes, tile width chosen for whole waves of 148 SMs
    p = capi.gemm_tile_plan(4096, 512)
    assert p["swapped"] and p["lane_tiles"] * p["col_tiles"] == 148
    p = capi.gemm_tile_plan(14336, 512)
    assert p["swapped"] and 0.9 <= p["lane_tiles"] * p["col_tiles"] / (2 * 148) <= 1.0
