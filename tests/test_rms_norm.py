"""rms_norm x norm-weight (-> Q8_0): the CPU oracle against the reference's vectors (no GPU), and the CUDA kernels
against the oracle through the C ABI (gpu)."""
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "rms_norm_ref_vectors.npz")


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def vectors():
    return np.load(GOLDEN)


def _cases(v):
    i = 0
    while f"x{i}" in v:
        for mode in (0, 1):
            e = 0
            while f"y{i}_m{mode}_e{e}" in v:
                yield i, mode, e, float(v["eps"][e])
                e += 1
        i += 1


# ---------------------------------------------------------------- oracle pinned (CPU) ----------------------------------------------------------------
def test_oracle_against_reference_vectors(oracle, vectors):
    v, n = vectors, 0
    for i, mode, e, eps in _cases(v):
        x, w = v[f"x{i}"], v[f"w{i}"]
        assert (_bits(oracle.rms_norm_mul(x, w, eps, mode)) == v[f"y{i}_m{mode}_e{e}"]).all(), (i, mode, e)
        assert (oracle.rms_norm_mul_q8_0(x, w, eps, mode) == v[f"q{i}_m{mode}_e{e}"]).all(), (i, mode, e)
        n += 1
    assert n >= 20
    for i in range(6):
        got = np.array([oracle.sum_squares(r) for r in v[f"x{i}"]], dtype=np.float32).view(np.uint32)
        assert (got == v[f"sumsq{i}"]).all()
    got = np.array([oracle.sqrtf_fast(float(t)) for t in v["sqrt_in"]], dtype=np.float32).view(np.uint32)
    assert (got == v["sqrt_fast_out"]).all()


def test_oracle_against_reference_in_place_build(oracle, reference):
    if reference is None or not reference.has_rms_norm:
        pytest.skip("oracle/_ref not built with the rms_norm helpers (reference tree absent)")
    rng = np.random.default_rng(5)
    for K in (32, 64, 128, 256, 1024, 2048, 4096):
        x = (rng.standard_normal((3, K)) * rng.uniform(0.01, 50.0)).astype(np.float32)
        w = rng.uniform(0.2, 2.0, K).astype(np.float32)
        for mode in (0, 1):
            assert (_bits(oracle.rms_norm_mul(x, w, 1e-5, mode)) == _bits(reference.rms_norm_mul(x, w, 1e-5, mode))).all()
            assert (oracle.rms_norm_mul_q8_0(x, w, 1e-5, mode) == reference.rms_norm_mul_q8_0(x, w, 1e-5, mode)).all()


def test_oracle_known_answers(oracle):
    # a row of equal values: sum = K v^2 exactly (powers of two), scale = 1 / sqrt(v^2 + eps)
    K = 256
    x = np.full((1, K), 2.0, dtype=np.float32)
    w = np.full(K, 0.5, dtype=np.float32)
    y = oracle.rms_norm_mul(x, w, 0.0, 0)
    assert (y == np.float32(0.5)).all()  # (2 * 0.5) * (1 / sqrt(4)) = 0.5
    blocks = oracle.rms_norm_mul_q8_0(x, w, 0.0, 0)
    assert (blocks[0, :, 2:].view(np.int8) == 127).all()
    # IEEE mode agrees with a float64 evaluation to rounding; the x86 formula is off by about 2^64
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 4096)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 4096).astype(np.float32)
    truth = x / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-5) * w
    assert np.abs(oracle.rms_norm_mul(x, w, 1e-5, 0) - truth).max() <= 1e-5 * np.abs(truth).max()
    ratio = oracle.rms_norm_mul(x, w, 1e-5, 0)[0, 0] / oracle.rms_norm_mul(x, w, 1e-5, 1)[0, 0]
    assert 2.0**63 < ratio < 2.0**65
    # the x86 formula's scales underflow fp16: every stored d is zero, the quants are still the rounded row
    b = oracle.rms_norm_mul_q8_0(x, w, 1e-5, 1)
    assert (b[:, :, :2] == 0).all() and (np.abs(b[:, :, 2:].view(np.int8)).max(axis=2) == 127).all()


def test_host_argument_checks(capi):
    lib = capi.lib
    # a null context is rejected before anything touches the GPU
    assert lib.nhb_rms_norm_mul(None, None, 32, None, 1e-5, 0, None, 32, 1, 32) != 0
    assert lib.nhb_rms_norm_mul_q8_0(None, None, 32, None, 1e-5, 0, None, 1, 32) != 0
    assert lib.nhb_rms_norm_mul_mat_batch(None, None, 0, None, 1e-5, 0, 0) != 0


# ---------------------------------------------------------------- CUDA against the oracle ----------------------------------------------------------------
@pytest.fixture(scope="module")
def ctx(capi):
    import torch

    c = capi.Context(0)
    c.use_torch_stream()
    yield c
    torch.cuda.synchronize()
    c.close()


@pytest.mark.gpu
def test_gpu_against_reference_vectors(ctx, vectors):
    import torch

    v = vectors
    for i, mode, e, eps in _cases(v):
        x = torch.from_numpy(v[f"x{i}"]).cuda()
        w = torch.from_numpy(v[f"w{i}"]).cuda()
        y = ctx.rms_norm_mul(x, w, eps, mode)
        b = ctx.rms_norm_mul_q8_0(x, w, eps, mode)
        torch.cuda.synchronize()
        assert (_bits(y.cpu().numpy()) == v[f"y{i}_m{mode}_e{e}"]).all(), (i, mode, e)
        assert (b.cpu().numpy() == v[f"q{i}_m{mode}_e{e}"]).all(), (i, mode, e)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K", [(1, 4096), (4, 4096), (7, 160), (33, 1024), (512, 4096), (3, 14336), (2, 51200), (0, 64)])
def test_gpu_against_oracle(ctx, oracle, M, K):
    import torch

    rng = np.random.default_rng(M * 131 + K)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.02, 30.0, (M, 1))).astype(np.float32)
    w = rng.uniform(0.1, 2.0, K).astype(np.float32)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    for mode in (0, 1):
        y = ctx.rms_norm_mul(xd, wd, 1e-5, mode)
        b = ctx.rms_norm_mul_q8_0(xd, wd, 1e-5, mode)
        torch.cuda.synchronize()
        if M == 0:
            continue
        assert (_bits(y.cpu().numpy()) == _bits(oracle.rms_norm_mul(x, w, 1e-5, mode))).all()
        assert (b.cpu().numpy() == oracle.rms_norm_mul_q8_0(x, w, 1e-5, mode)).all()


@pytest.mark.gpu
def test_gpu_strided_rows(ctx, oracle):
    import torch

    rng = np.random.default_rng(9)
    M, K, ld = 5, 512, 640
    xs = rng.standard_normal((M, ld)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, K).astype(np.float32)
    xd = torch.from_numpy(xs).cuda()
    yd = torch.full((M, ld), -7.0, device="cuda")
    ctx.rms_norm_mul(xd[:, :K], torch.from_numpy(w).cuda(), 1e-6, 0, y=yd[:, :K])
    torch.cuda.synchronize()
    got = yd.cpu().numpy()
    assert (_bits(got[:, :K]) == _bits(oracle.rms_norm_mul(xs[:, :K], w, 1e-6, 0))).all()
    assert (got[:, K:] == -7.0).all()


@pytest.mark.gpu
@pytest.mark.parametrize("M,K", [(1, 1024), (3, 1024), (4, 1024), (6, 1024), (40, 1024), (1, 4096), (2, 4096), (4, 4096), (1, 14336), (4, 14336)])
def test_gpu_norm_feeding_mul_mats(ctx, capi, oracle, M, K):
    """Fused producer -> projections (norm inside the GEMV's prologue, as a separate quantising kernel when the rows
    do not fit its shared memory, through a scratch buffer for the GEMM): bit-identical to the two-call composition,
    and equal to the oracle's rms_norm_mul followed by its Q8-arithmetic mul_mat."""
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    rng = np.random.default_rng(77 + M + K)
    x = (rng.standard_normal((M, K)) * 3.0).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, K).astype(np.float32)
    w1, w2 = synth.make_weight(200, K, 1), synth.make_weight(72, K, 2)
    h1, h2 = ctx.upload(w1), ctx.upload(w2)
    xd, nwd = torch.from_numpy(x).cuda(), torch.from_numpy(nw).cuda()
    y1, y2 = torch.zeros((M, 200), device="cuda"), torch.zeros((M, 72), device="cuda")
    ctx.rms_norm_mul_mat_batch([(h1, xd, y1), (h2, xd, y2)], nwd, 1e-5)
    z1, z2 = torch.zeros((M, 200), device="cuda"), torch.zeros((M, 72), device="cuda")
    normed = ctx.rms_norm_mul(xd, nwd, 1e-5)
    ctx.mul_mat_batch([(h1, normed, z1), (h2, normed, z2)])
    torch.cuda.synchronize()
    assert torch.equal(y1, z1) and torch.equal(y2, z2)
    n_ref = oracle.rms_norm_mul(x, nw, 1e-5, 0)
    for w, y in ((w1, y1), (w2, y2)):
        ref = oracle.mul_mat(po.Q8ACT_LANES, w, n_ref)
        err = np.abs(y.cpu().numpy() - ref).max() / np.abs(ref).max()
        assert err <= 1e-4, err  # f32 tolerance of the mul_mat path: max|err| / max|ref| <= 1e-4
    h1.free()
    h2.free()


@pytest.mark.gpu
def test_gpu_norm_batch_rejects_mixed_inputs(ctx, capi):
    import torch

    from nihilus_b200 import synth

    h = ctx.upload(synth.make_weight(64, 256, 3))
    xa, xb = torch.zeros((1, 256), device="cuda"), torch.zeros((1, 256), device="cuda")
    nw = torch.ones(256, device="cuda")
    y = torch.zeros((1, 64), device="cuda")
    with pytest.raises(capi.NhbError):
        ctx.rms_norm_mul_mat_batch([(h, xa, y), (h, xb, y)], nw, 1e-5)
    with pytest.raises(capi.NhbError):
        ctx.rms_norm_mul(torch.zeros((1, 48), device="cuda"), torch.ones(48, device="cuda"), 1e-5)  # K % 32 != 0
    with pytest.raises(capi.NhbError):
        ctx.rms_norm_mul(xa, nw, 1e-5, sqrt_mode=7)
    h.free()
