"""Parity of the tensor-core prefill GEMM at the shapes the benchmark times (needs a B200).

The 512- and 2048-token shapes of the LLaMA-3-8B projections take the token-on-lanes orientation with wide tiles,
kernel instantiations the small-shape tests never reach.  Each case first asserts the tile plan, so that a change of
the planner cannot silently move the test onto another kernel, then compares with the CPU oracle
(include/nihilus-incl/cpu/avx_2.hpp:4749-4780 row dot, :4926-4963 loop nest) on a subset of weight rows that
touches every column tile, every epilogue column group and both ragged edges, over all tokens.  Rows of a mul_mat
are independent, so oracle(w[idx], x) is the reference for y[:, idx].
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-4  # max|err| / max|ref|


def _rel(y, ref):
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.fixture(scope="module")
def ctx(capi):
    c = capi.Context(0)
    c.use_torch_stream()
    yield c
    c.close()


def subset_rows(N: int, tile: int, stride: int = 29) -> np.ndarray:
    """Every `stride`-th row (coprime to the 8-column units and to every tile width), the whole first and last tile."""
    idx = set(range(0, N, stride))
    idx.update(range(0, min(N, tile)))
    idx.update(range(max(0, N - tile), N))
    return np.array(sorted(idx), dtype=np.int64)


def check_against_oracle(oracle, po, w, x, y, tile):
    idx = subset_rows(w.shape[0], tile)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w[idx], x)
    got = y[:, idx]
    assert _rel(got, ref) <= TOL
    assert _rel(got, oracle.mul_mat(po.Q8ACT_F64, w[idx], x)) <= TOL
    return _rel(got, ref)


# (N, K, M) -> the plan the benchmarked kernel must have: token-on-lanes, tile width
BENCH_SHAPES = [
    ((14336, 4096, 512), 208),  # ffn_gate / ffn_up
    ((4096, 14336, 512), 112),  # ffn_down
    ((14336, 4096, 2048), 224),  # ffn_gate / ffn_up at 2048 tokens
    ((4096, 4096, 2048), 112),  # attn_q at 2048 tokens
    ((128256, 4096, 512), 208),  # lm_head
]


@pytest.mark.parametrize("shape,tile", BENCH_SHAPES)
def test_benchmarked_prefill_instantiations_match_the_oracle(capi, ctx, oracle, shape, tile):
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    N, K, M = shape
    plan = capi.gemm_tile_plan(N, M)
    assert plan["swapped"] and plan["tile_cols"] == tile, plan
    w = synth.make_weight(N, K, 20253000 + N + M)
    x = synth.make_activation(M, K, 20253001 + K + M)
    h = ctx.upload(w)
    xd = torch.from_numpy(x).cuda()
    y = torch.full((M, N), float("nan"), device="cuda")
    ctx.mul_mat(h, xd, y, kernel=capi.KERNEL_GEMM_TC)
    ctx.sync()
    yy = y.cpu().numpy()
    assert np.isfinite(yy).all()  # every element was written
    check_against_oracle(oracle, po, w, x, yy, tile)
    # AUTO takes the same kernel for M > 8: same bits
    y2 = torch.zeros((M, N), device="cuda")
    ctx.mul_mat(h, xd, y2)
    ctx.sync()
    assert torch.equal(y, y2)
    h.free()


@pytest.mark.parametrize("N,K,M", [(14331, 512, 500), (4099, 4096, 500), (7001, 1024, 200), (5003, 14336, 500)])
def test_ragged_shapes_in_the_token_on_lanes_orientation(capi, ctx, oracle, N, K, M):
    """N not a multiple of the tile width and M not a multiple of 128: ragged on both sides, padding untouched."""
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    plan = capi.gemm_tile_plan(N, M)
    assert plan["swapped"] and N % plan["tile_cols"] != 0 and M % 128 != 0, plan
    w = synth.make_weight(N, K, 977 + N)
    x = synth.make_activation(M, K, 978 + M)
    h = ctx.upload(w)
    xd = torch.from_numpy(x).cuda()
    y = torch.full((M, N + 5), -7.0, device="cuda")
    capi._check(capi.lib.nhb_mul_mat(ctx.handle, h.handle, xd.data_ptr(), K, y.data_ptr(), N + 5, M, capi.ACT_Q8, capi.KERNEL_GEMM_TC), ctx.handle)
    ctx.sync()
    yy = y.cpu().numpy()
    assert (yy[:, N:] == -7.0).all()
    check_against_oracle(oracle, po, w, x, yy[:, :N], plan["tile_cols"])
    h.free()


@pytest.mark.parametrize("N,K,M", [(14336, 4096, 512), (4096, 14336, 512)])
def test_wide_tile_row_shards_are_bit_identical_to_one_gpu(capi, ctx, N, K, M):
    """Shards of 1/2 and 1/4 of the rows plan other tile widths; every element still carries the unsharded bits."""
    import torch

    from nihilus_b200 import synth

    w = synth.make_weight(N, K, 4000 + N)
    xd = torch.from_numpy(synth.make_activation(M, K, 4001 + K)).cuda()
    h = ctx.upload(w)
    full = torch.zeros((M, N), device="cuda")
    ctx.mul_mat(h, xd, full, kernel=capi.KERNEL_GEMM_TC)
    ctx.sync()
    h.free()
    for world in (2, 4):
        widths = set()
        y = torch.zeros((M, N), device="cuda")
        for r in range(world):
            c = capi.Context(0, r, world)
            c.use_torch_stream()
            hr = c.upload(w)
            widths.add(capi.gemm_tile_plan(hr.n1 - hr.n0, M)["tile_cols"])
            c.mul_mat(hr, xd, y, kernel=capi.KERNEL_GEMM_TC)
            c.sync()
            hr.free()
            c.close()
        assert torch.equal(y, full), (world, widths)


@pytest.mark.parametrize("K", [4096, 14336])
@pytest.mark.parametrize("M", [9, 16, 32])
def test_few_tokens_split_k_over_ctas_and_every_split_gives_the_same_bits(capi, ctx, oracle, K, M):
    """Up to 32 tokens the GEMM sums K in chunks whose totals are added in ascending order, so that a tile's chunks can be
    dealt to several CTAs when the weight has fewer tiles than the GPU has SMs.  An unsharded weight of 148 tiles is walked
    by one CTA per tile; its 1/8 shards (19 tiles) by 4 to 7 CTAs per tile; the shards' rows carry the unsharded bits."""
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    N = 148 * 128
    w = synth.make_weight(N, K, 4100 + K)
    x = synth.make_activation(M, K, 4101 + M)
    xd = torch.from_numpy(x).cuda()
    h = ctx.upload(w)
    full = torch.zeros((M, N), device="cuda")
    ctx.mul_mat(h, xd, full, kernel=capi.KERNEL_GEMM_TC)
    ctx.mul_mat(h, xd, full, kernel=capi.KERNEL_GEMM_TC)  # a second launch finds the arrival counters back at zero
    ctx.sync()
    h.free()
    rows = slice(0, N, 7)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w[rows], x)
    got = full.cpu().numpy()
    assert float(np.abs(got[:, rows] - ref).max() / np.abs(ref).max()) <= TOL
    y = torch.zeros((M, N), device="cuda")
    for r in range(8):
        c = capi.Context(0, r, 8)
        c.use_torch_stream()
        hr = c.upload(w)
        for _ in range(2):
            c.mul_mat(hr, xd, y, kernel=capi.KERNEL_GEMM_TC)
        c.sync()
        hr.free()
        c.close()
    assert torch.equal(y, full)


def test_operand_planes_rebuilt_per_call_give_the_same_bits_as_kept_ones(capi, oracle):
    """Option gemm_keep_planes = 0: no fp16 copy stays with the weight; q, k, v sharing one input still quantise it once."""
    import torch

    from nihilus_b200 import synth

    M, K = 200, 4096
    ws = [synth.make_weight(n, K, 4200 + n) for n in (4096, 1024, 1031)]
    xd = torch.from_numpy(synth.make_activation(M, K, 4203)).cuda()
    outs = []
    for keep in (1, 0):
        c = capi.Context(0)
        c.use_torch_stream()
        c.set_option("gemm_keep_planes", keep)
        hs = [c.upload(w) for w in ws]
        ys = [torch.zeros((M, h.N), device="cuda") for h in hs]
        for _ in range(2):
            c.mul_mat_batch([(h, xd, y) for h, y in zip(hs, ys)], kernel=capi.KERNEL_GEMM_TC)
        c.sync()
        outs.append([y.clone() for y in ys])
        for h in hs:
            h.free()
        c.close()
    for a, b in zip(*outs):
        assert torch.equal(a, b)
