"""Parity of the CUDA path against the CPU oracle, through the C ABI (needs a B200)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-4  # max|err| / max|ref| for f32 outputs; per-block int32 dots must be exact


def _rel(y, ref):
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.fixture(scope="module")
def ctx(capi):
    c = capi.Context(0)
    c.use_torch_stream()
    yield c
    c.close()


@pytest.fixture(scope="module")
def torch_mod():
    import torch

    return torch


def _case(synth, N, K, M, seed):
    return synth.make_weight(N, K, seed), synth.make_activation(M, K, seed + 1)


def _run(ctx, torch, w_handle, x, **kw):
    xd = torch.from_numpy(x).cuda()
    y = ctx.mul_mat(w_handle, xd, **kw)
    ctx.sync()
    return y.cpu().numpy()


def test_loaded_library_is_ours(capi):
    assert "libnihilus_b200.so" in open("/proc/self/maps").read()


def test_upload_repack_round_trip(capi, ctx, oracle):
    from nihilus_b200 import synth

    for N, K in ((37, 96), (128, 4096), (5, 14336)):
        w = synth.make_weight(N, K, 5)
        h = ctx.upload(w)
        assert (h.download() == w).all()
        assert h.bytes_q8 == N * (K // 32) * 34
        h.free()


def test_quantiser_bit_exact(capi, ctx, oracle, torch_mod):
    torch = torch_mod
    rng = np.random.default_rng(31)
    x = rng.standard_normal((5, 4096)).astype(np.float32)
    x[0, :32] = 0.0
    x[1, :64] *= 1e-6
    x[2, 100] = 1e4
    x[3, :32] = [0.5 * i for i in range(32)]  # exact ties after scaling by 127/15.5
    q, d = ctx.quantize(torch.from_numpy(x).cuda())
    ctx.sync()
    blocks = oracle.quantize_rows(x)
    want_q = blocks[:, :, 2:].view(np.int8).reshape(5, 4096)
    want_d = blocks[:, :, :2].copy().view(np.float16).astype(np.float32).reshape(5, 128)
    assert (q.cpu().numpy() == want_q).all()
    assert (d.cpu().numpy().view(np.uint32) == want_d.view(np.uint32)).all()


@pytest.mark.parametrize("N,K", [(8, 32), (9, 64), (33, 96), (64, 256), (17, 1024), (40, 2048), (31, 4096), (6, 14336)])
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8])
def test_small_shapes_q8(capi, ctx, oracle, torch_mod, N, K, M):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    w, x = _case(synth, N, K, M, 1000 + N + K + M)
    h = ctx.upload(w)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
    y = _run(ctx, torch_mod, h, x)
    assert _rel(y, ref) <= TOL
    # exact integer block dots
    dots = ctx.block_dots(h, torch_mod.from_numpy(x).cuda())
    ctx.sync()
    assert (dots.cpu().numpy() == oracle.block_dots(w, x)).all()
    h.free()


@pytest.mark.parametrize("kernel_name", ["KERNEL_GEMV_LDG", "KERNEL_GEMV_STREAM", "KERNEL_GEMV_ROWS"])
@pytest.mark.parametrize("N,K", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_llama_shapes_m1_both_gemv_kernels(capi, ctx, oracle, torch_mod, kernel_name, N, K):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    w, x = _case(synth, N, K, 1, 20250000 + N + K)
    h = ctx.upload(w)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
    y = _run(ctx, torch_mod, h, x, kernel=getattr(capi, kernel_name))
    assert _rel(y, ref) <= TOL
    truth = oracle.mul_mat(po.Q8ACT_F64, w, x)
    assert _rel(y, truth) <= TOL
    h.free()


def test_lm_head_full_size(capi, ctx, oracle, torch_mod):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    N, K = 128256, 4096
    w, x = _case(synth, N, K, 1, 20252007)
    h = ctx.upload(w)
    y = _run(ctx, torch_mod, h, x)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
    assert _rel(y, ref) <= TOL
    # size-independent property: permuting weight rows permutes outputs, bit for bit
    perm = np.random.default_rng(1).permutation(N)
    h2 = ctx.upload(w[perm])
    y2 = _run(ctx, torch_mod, h2, x)
    assert (y2.view(np.uint32) == y[:, perm].view(np.uint32)).all()
    h.free()
    h2.free()


@pytest.mark.parametrize("M", [1, 2, 4, 7, 8, 11])
def test_multi_row_stream_and_ldg_agree(capi, ctx, oracle, torch_mod, M):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    for N, K in ((512, 4096), (256, 14336)):
        w, x = _case(synth, N, K, M, 77 + M)
        h = ctx.upload(w)
        ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
        ys = _run(ctx, torch_mod, h, x, kernel=capi.KERNEL_GEMV_STREAM)
        yl = _run(ctx, torch_mod, h, x, kernel=capi.KERNEL_GEMV_LDG)
        yr = _run(ctx, torch_mod, h, x, kernel=capi.KERNEL_GEMV_ROWS)
        assert _rel(ys, ref) <= TOL and _rel(yl, ref) <= TOL and _rel(yr, ref) <= TOL
        h.free()


@pytest.mark.parametrize("N,K,M", [(128, 256, 9), (128, 256, 16), (300, 512, 17), (130, 1024, 33), (256, 4096, 64), (1000, 4096, 100),
                                   (384, 4096, 128), (512, 4096, 200), (256, 14336, 257), (640, 4096, 512), (130, 64, 20), (1000, 192, 130),
                                   (4100, 256, 300), (37, 128, 1000)])
def test_tensor_core_gemm_prefill(capi, ctx, oracle, torch_mod, N, K, M):
    """tcgen05 GEMM: exact int block dots on the tensor cores, f32 outputs within 1e-4 of the oracle; AUTO picks it for M > 8."""
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    w, x = _case(synth, N, K, M, 31337 + N + M)
    h = ctx.upload(w)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
    y = _run(ctx, torch_mod, h, x, kernel=capi.KERNEL_GEMM_TC)
    assert _rel(y, ref) <= TOL
    assert _rel(y, oracle.mul_mat(po.Q8ACT_F64, w, x)) <= TOL
    ya = _run(ctx, torch_mod, h, x)  # AUTO
    assert (ya.view(np.uint32) == y.view(np.uint32)).all()
    # GEMV passes over the same rows agree to the tolerance as well (different summation order)
    yg = _run(ctx, torch_mod, h, x[:8], kernel=capi.KERNEL_GEMV_ROWS)
    assert _rel(y[:8], yg) <= TOL
    h.free()


def test_tensor_core_gemm_ragged_output_and_sharding(capi, ctx, oracle, torch_mod):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    torch = torch_mod
    N, K, M = 777, 4096, 48
    w, x = _case(synth, N, K, M, 4711)
    xd = torch.from_numpy(x).cuda()
    ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
    full = None
    for world in (1, 2, 3):
        y = torch.full((M, N + 3), -7.0, device="cuda")
        for r in range(world):
            c = capi.Context(0, r, world)
            c.use_torch_stream()
            hr = c.upload(w)
            capi._check(capi.lib.nhb_mul_mat(c.handle, hr.handle, xd.data_ptr(), K, y.data_ptr(), N + 3, M, capi.ACT_Q8, capi.KERNEL_GEMM_TC), c.handle)
            c.sync()
            hr.free()
            c.close()
        yy = y.cpu().numpy()
        assert (yy[:, N:] == -7.0).all()
        assert _rel(yy[:, :N], ref) <= TOL
        if full is None:
            full = yy.copy()
        assert (yy.view(np.uint32) == full.view(np.uint32)).all()  # row shards are bit-identical to one GPU


@pytest.mark.parametrize("N,K,M", [(64, 256, 1), (100, 4096, 3), (32, 14336, 2), (9, 96, 5), (3700, 4096, 2), (3600, 14336, 1), (5000, 512, 7)])
def test_f32_activation_mode(capi, ctx, oracle, torch_mod, N, K, M):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    w, x = _case(synth, N, K, M, 4242 + N)
    h = ctx.upload(w)
    ref = oracle.mul_mat(po.F32ACT_EVAL, w, x)
    y = _run(ctx, torch_mod, h, x, act_mode=capi.ACT_F32)
    assert _rel(y, ref) <= TOL
    assert _rel(y, oracle.mul_mat(po.F32ACT_PROMPT, w, x)) <= TOL
    h.free()


def test_ragged_leading_dimensions_and_untouched_padding(capi, ctx, oracle, torch_mod):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    torch = torch_mod
    N, K, M = 130, 4096, 3
    w, x = _case(synth, N, K, M, 9)
    h = ctx.upload(w)
    xd = torch.full((M, K + 64), 7.0, device="cuda")
    xd[:, :K] = torch.from_numpy(x).cuda()
    yd = torch.full((M, N + 6), -3.0, device="cuda")
    capi._check(capi.lib.nhb_mul_mat(ctx.handle, h.handle, xd.data_ptr(), K + 64, yd.data_ptr(), N + 6, M, capi.ACT_Q8, capi.KERNEL_AUTO), ctx.handle)
    ctx.sync()
    y = yd.cpu().numpy()
    assert _rel(y[:, :N], oracle.mul_mat(po.Q8ACT_LANES, w, x)) <= TOL
    assert (y[:, N:] == -3.0).all()
    h.free()


def test_empty_inputs_and_argument_errors(capi, ctx, torch_mod):
    from nihilus_b200 import synth

    torch = torch_mod
    w = synth.make_weight(16, 64, 3)
    h = ctx.upload(w)
    x0 = torch.zeros((0, 64), device="cuda")
    assert ctx.mul_mat(h, x0).shape == (0, 16)
    hz = ctx.upload(w[:0])  # a weight with no rows
    y = ctx.mul_mat(hz, torch.zeros((2, 64), device="cuda"))
    ctx.sync()
    assert y.shape == (2, 0)
    x = torch.zeros((1, 64), device="cuda")
    yb = torch.zeros((1, 16), device="cuda")
    lib = capi.lib
    assert lib.nhb_mul_mat(ctx.handle, h.handle, None, 64, yb.data_ptr(), 16, 1, 0, 0) == capi.ERR_ARG
    assert lib.nhb_mul_mat(ctx.handle, h.handle, x.data_ptr(), 32, yb.data_ptr(), 16, 1, 0, 0) == capi.ERR_ARG  # ldx < K
    assert lib.nhb_mul_mat(ctx.handle, h.handle, x.data_ptr(), 64, yb.data_ptr(), 8, 1, 0, 0) == capi.ERR_ARG  # ldy < N
    assert lib.nhb_mul_mat(ctx.handle, h.handle, x.data_ptr(), 64, yb.data_ptr(), 16, -1, 0, 0) == capi.ERR_ARG
    assert lib.nhb_mul_mat(ctx.handle, h.handle, x.data_ptr(), 64, yb.data_ptr(), 16, 1, 9, 0) == capi.ERR_ARG  # mode
    assert lib.nhb_mul_mat(ctx.handle, h.handle, x.data_ptr() + 4, 64, yb.data_ptr(), 16, 1, 0, 0) == capi.ERR_ARG  # misaligned
    assert lib.nhb_mul_mat(ctx.handle, h.handle, x.data_ptr(), 64, yb.data_ptr(), 16, 1, 0, 99) == capi.ERR_ARG  # kernel id
    assert lib.nhb_mul_mat(ctx.handle, h.handle, x.data_ptr(), 64, x.data_ptr() + 128, 16, 1, 0, 0) == capi.ERR_ARG  # y inside x
    assert lib.nhb_mul_mat(ctx.handle, h.handle, x.data_ptr(), 64, yb.data_ptr(), 16, 1, 0, capi.KERNEL_GEMV_STREAM) == capi.ERR_UNSUPPORTED
    assert "K" in capi.last_error(ctx.handle)
    import ctypes as C

    out = C.c_void_p()
    assert lib.nhb_weight_upload_q8_0(ctx.handle, w.ctypes.data, 16, 48, C.byref(out)) == capi.ERR_ARG  # K % 32
    ctx.sync()  # the context is still usable
    h.free()
    hz.free()


@pytest.mark.parametrize("kernel_name", ["KERNEL_GEMV_STREAM", "KERNEL_GEMV_ROWS", "KERNEL_AUTO"])
def test_batched_launch_equals_single_launches(capi, ctx, oracle, torch_mod, kernel_name):
    from nihilus_b200 import synth

    torch = torch_mod
    kern = getattr(capi, kernel_name)
    shapes = [(4096, 4096), (1024, 4096), (1024, 4096), (640, 14336)]
    hs, xs, singles = [], [], []
    for i, (N, K) in enumerate(shapes):
        w = synth.make_weight(N, K, 300 + i)
        hs.append(ctx.upload(w))
        xs.append(torch.from_numpy(synth.make_activation(1, K, 400 + i)).cuda())
        singles.append(ctx.mul_mat(hs[-1], xs[-1], kernel=kern))
    ys = [torch.zeros((1, N), device="cuda") for N, _ in shapes]
    ctx.mul_mat_batch([(h, x, y) for h, x, y in zip(hs, xs, ys)], kernel=kern)
    ctx.sync()
    for a, b in zip(singles, ys):
        assert torch.equal(a, b)
    for h in hs:
        h.free()


def test_rows_kernel_options_do_not_change_results(capi, oracle, torch_mod):
    """Grid size (CTAs per SM), register cap and separate activation quantisation leave every bit unchanged."""
    from nihilus_b200 import synth

    torch = torch_mod
    base = None
    w1 = synth.make_weight(1500, 4096, 61)
    w2 = synth.make_weight(700, 4096, 62)
    w3 = synth.make_weight(300, 14336, 63)
    x1 = torch.from_numpy(synth.make_activation(2, 4096, 64)).cuda()
    x3 = torch.from_numpy(synth.make_activation(2, 14336, 65)).cuda()
    for cps, db, cl in ((2, 0, 1), (3, 0, 1), (4, 0, 1), (2, 1, 1), (3, 1, 1), (3, 0, 2), (3, 0, 4), (2, 0, 8), (2, 1, 4)):
        for preq in (0, 1):
            for pdl in (0, 1):
                c = capi.Context(0)
                c.use_torch_stream()
                c.set_option("rows_double_buffer", db)
                c.set_option("rows_cluster", cl)
                c.set_option("rows_ctas_per_sm", cps)
                c.set_option("prequantize", preq)
                c.set_option("pdl", pdl)
                hs = [c.upload(w1), c.upload(w2), c.upload(w3)]
                ys = [torch.zeros((2, 1500), device="cuda"), torch.zeros((2, 700), device="cuda"), torch.zeros((2, 300), device="cuda")]
                for _ in range(2):  # back-to-back launches exercise the programmatic-dependent-launch path
                    c.mul_mat_batch([(hs[0], x1, ys[0]), (hs[1], x1, ys[1]), (hs[2], x3, ys[2])], kernel=capi.KERNEL_GEMV_ROWS)
                c.sync()
                got = [y.cpu().numpy().copy() for y in ys]
                if base is None:
                    base = got
                for a, b in zip(base, got):
                    assert (a.view(np.uint32) == b.view(np.uint32)).all(), (cps, db, cl, preq, pdl)
                for h in hs:
                    h.free()
                c.close()
    from oracle import pyoracle as po

    assert _rel(base[0], oracle.mul_mat(po.Q8ACT_LANES, w1, x1.cpu().numpy())) <= TOL
    assert _rel(base[2], oracle.mul_mat(po.Q8ACT_LANES, w3, x3.cpu().numpy())) <= TOL


def test_wide_launch_cta_shape_is_bit_identical(capi, oracle, torch_mod):
    """Launches with at least 24 rows per SM use one 24-warp CTA per SM; the result must not depend on that choice."""
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    torch = torch_mod
    w1, w2 = synth.make_weight(4100, 512, 71), synth.make_weight(1333, 512, 72)
    outs = []
    for M in (1, 3):
        x = torch.from_numpy(synth.make_activation(M, 512, 73 + M)).cuda()
        per_shape = []
        for fat in (0, 1):
            c = capi.Context(0)
            c.use_torch_stream()
            c.set_option("rows_fat_ctas", fat)
            hs = [c.upload(w1), c.upload(w2)]
            ys = [torch.zeros((M, 4100), device="cuda"), torch.zeros((M, 1333), device="cuda")]
            for _ in range(2):
                c.mul_mat_batch([(hs[0], x, ys[0]), (hs[1], x, ys[1])])
            c.sync()
            per_shape.append([y.cpu().numpy().copy() for y in ys])
            for h in hs:
                h.free()
            c.close()
        for a, b in zip(*per_shape):
            assert (a.view(np.uint32) == b.view(np.uint32)).all()
        assert _rel(per_shape[1][0], oracle.mul_mat(po.Q8ACT_LANES, w1, x.cpu().numpy())) <= TOL
        assert _rel(per_shape[1][1], oracle.mul_mat(po.Q8ACT_LANES, w2, x.cpu().numpy())) <= TOL
        outs.append(per_shape)


def test_long_rows_item_parallel_kernel_is_bit_identical(capi, oracle, torch_mod):
    """Rows longer than 4096 in a wide launch are split into 4 KB items over the warps of a CTA; item totals are
    added in the same order as in the one-warp-per-row kernels, so the three kernels agree bit for bit."""
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    torch = torch_mod
    N, K = 3700, 14336
    w = synth.make_weight(N, K, 81)
    for M in (1, 4):
        x = torch.from_numpy(synth.make_activation(M, K, 82 + M)).cuda()
        got = []
        for fat, split in ((0, 0), (1, 0), (1, 1)):
            c = capi.Context(0)
            c.use_torch_stream()
            c.set_option("rows_fat_ctas", fat)
            c.set_option("rows_split_long", split)
            h = c.upload(w)
            y = torch.zeros((M, N), device="cuda")
            for _ in range(2):
                c.mul_mat(h, x, y)
            c.sync()
            got.append(y.cpu().numpy().copy())
            h.free()
            c.close()
        assert (got[0].view(np.uint32) == got[1].view(np.uint32)).all()
        assert (got[0].view(np.uint32) == got[2].view(np.uint32)).all()
        assert _rel(got[2], oracle.mul_mat(po.Q8ACT_LANES, w, x.cpu().numpy())) <= TOL


def test_emulated_row_shards_are_bit_identical_to_one_gpu(capi, ctx, oracle, torch_mod):
    """world = 2, 4 and 3 (uneven) emulated as several contexts on this GPU: concatenated slices == unsharded."""
    from nihilus_b200 import synth

    torch = torch_mod
    N, K, M = 1030, 4096, 2
    w, x = _case(synth, N, K, M, 555)
    h = ctx.upload(w)
    full = _run(ctx, torch, h, x)
    h.free()
    xd = torch.from_numpy(x).cuda()
    for world in (2, 3, 4):
        y = torch.zeros((M, N), device="cuda")
        for r in range(world):
            c = capi.Context(0, r, world)
            c.use_torch_stream()
            hr = c.upload(w)
            assert (hr.n0, hr.n1) == capi.shard_rows(N, world, r)
            c.mul_mat(hr, xd, y)
            c.sync()
            hr.free()
            c.close()
        assert (y.cpu().numpy().view(np.uint32) == full.view(np.uint32)).all()


def test_graph_replay_and_determinism(capi, oracle, torch_mod):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    torch = torch_mod
    N, K = 2048, 4096
    w, x = _case(synth, N, K, 1, 808)
    side = torch.cuda.Stream()  # the legacy default stream cannot be captured
    with torch.cuda.stream(side):
        ctx = capi.Context(0)
        ctx.use_torch_stream()
        h = ctx.upload(w)
        xd = torch.from_numpy(x).cuda()
        y = torch.zeros((1, N), device="cuda")
        ctx.mul_mat(h, xd, y)
        ctx.sync()
        first = y.clone()
        ctx.graph_begin()
        for _ in range(3):
            ctx.mul_mat(h, xd, y)
        g = ctx.graph_end()
        y.zero_()
        g.launch()
        g.launch()
        ctx.sync()
        assert torch.equal(first, y)
        assert _rel(y.cpu().numpy(), oracle.mul_mat(po.Q8ACT_LANES, w, x)) <= TOL
        g.free()
        h.free()
        ctx.close()


def test_host_buffer_entry_point(capi, ctx, oracle):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    N, K, M = 300, 4096, 2
    w, x = _case(synth, N, K, M, 99)
    h = ctx.upload(w)
    y = ctx.mul_mat_host(h, x)
    assert _rel(y, oracle.mul_mat(po.Q8ACT_LANES, w, x)) <= TOL
    h.free()


@pytest.mark.gpu
def test_gemm_batch_sharing_its_input_quantises_once_and_is_bit_identical(ctx, capi):
    """q/k/v-style batch through the tensor-core GEMM: the shared input is quantised by the first op only; results are
    the bits of three separate calls, also when a different input sits between two uses of the same one."""
    import torch

    from nihilus_b200 import synth

    K, M = 512, 40
    ws = [ctx.upload(synth.make_weight(n, K, 300 + n)) for n in (256, 128, 192)]
    xa = torch.from_numpy(synth.make_activation(M, K, 31)).cuda()
    xb = torch.from_numpy(synth.make_activation(M, K, 32)).cuda()
    single = []
    for w, x in zip(ws, (xa, xa, xb)):
        y = torch.zeros((M, w.N), device="cuda")
        ctx.mul_mat(w, x, y, kernel=capi.KERNEL_GEMM_TC)
        single.append(y)
    ctx.sync()
    l0 = ctx.launches
    ys = [torch.zeros((M, w.N), device="cuda") for w in ws]
    ctx.mul_mat_batch([(ws[0], xa, ys[0]), (ws[1], xa, ys[1]), (ws[2], xb, ys[2])], kernel=capi.KERNEL_GEMM_TC)
    ctx.sync()
    assert ctx.launches - l0 == 3 + 2  # three GEMMs, two quantisations
    for a, b in zip(single, ys):
        assert torch.equal(a, b)
    zs = [torch.zeros((M, w.N), device="cuda") for w in ws]
    ctx.mul_mat_batch([(ws[0], xa, zs[0]), (ws[2], xb, zs[2]), (ws[1], xa, zs[1])], kernel=capi.KERNEL_GEMM_TC)
    ctx.sync()
    for a, b in zip(single, zs):
        assert torch.equal(a, b)
    for w in ws:
        w.free()


@pytest.mark.gpu
@pytest.mark.parametrize("N,K,M", [(4096, 4096, 8), (1031, 4096, 5), (300, 512, 7), (14336, 4096, 6), (64, 32, 8)])
def test_passes_of_up_to_eight_rows_are_bit_identical_to_passes_of_four(ctx, capi, oracle, N, K, M):
    """5 to 8 tokens go through the decode GEMV in one pass (rows of one 4 KB item); the values are those of the
    4-row passes -- the per-row arithmetic does not depend on how many rows share a pass -- and match the oracle."""
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    w = synth.make_weight(N, K, 500 + N)
    x = synth.make_activation(M, K, 501 + M)
    h = ctx.upload(w)
    xd = torch.from_numpy(x).cuda()
    y8 = torch.zeros((M, N), device="cuda")
    l0 = ctx.launches
    ctx.mul_mat(h, xd, y8, kernel=capi.KERNEL_GEMV_ROWS)
    ctx.sync()
    assert ctx.launches - l0 == 1
    ctx.set_option("prequantize", 1)  # the separate quantiser keeps passes of four
    y4 = torch.zeros((M, N), device="cuda")
    ctx.mul_mat(h, xd, y4, kernel=capi.KERNEL_GEMV_ROWS)
    ctx.sync()
    ctx.set_option("prequantize", 0)
    assert torch.equal(y8, y4)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
    assert np.abs(y8.cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()
    h.free()
