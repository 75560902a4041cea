"""Seeded random shapes through the public entry points, every result against the CPU oracle (needs a B200).

The other parity files pin the benchmarked shapes and the edge cases one by one; this one walks the space between them:
odd row counts, every K the kernels claim to take (multiples of 32; the GEMM needs 64), token counts on both sides of the
GEMV / GEMM switch and of the GEMM's 32-token rule, ragged leading dimensions, batches that share an input, emulated row
shards, the fused norm and the fused SwiGLU / residual tails.  Seeds are fixed: a failure names its case."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-4  # max|err| / max|ref|


def _rel(got, ref):
    return float(np.abs(got - ref).max() / max(float(np.abs(ref).max()), 1e-30))


def _cases(n, seed):
    rng = np.random.default_rng(seed)
    for i in range(n):
        K = int(rng.choice([32, 64, 96, 256, 1024, 2048, 4096, 4160, 8192]))
        N = int(rng.integers(1, 3000))
        M = int(rng.choice([1, 2, 3, 4, 5, 7, 8, 9, 15, 16, 17, 31, 32, 33, 48, 64, 65, 100, 128, 129, 130]))
        yield i, N, K, M, int(rng.integers(0, 2 ** 31))


@pytest.mark.parametrize("case,N,K,M,seed", list(_cases(36, 20251)))
def test_mul_mat_of_a_random_shape_matches_the_oracle(capi, oracle, case, N, K, M, seed):
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    rng = np.random.default_rng(seed)
    w = synth.make_weight(N, K, seed % 100000)
    x = (synth.make_activation(M, K, seed % 99991) * float(rng.choice([0.01, 1.0, 37.0]))).astype(np.float32)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w, x, threads=8)
    pad_x, pad_y = int(rng.choice([0, 4, 12])), int(rng.integers(0, 9))
    xd = torch.zeros((M, K + pad_x), device="cuda")
    xd[:, :K] = torch.from_numpy(x).cuda()
    world = int(rng.choice([1, 1, 2, 3, 8]))
    y = torch.full((M, N + pad_y), -7.0, device="cuda")
    for r in range(world):
        c = capi.Context(0, r, world)
        c.use_torch_stream()
        h = c.upload(w)
        capi._check(capi.lib.nhb_mul_mat(c.handle, h.handle, xd.data_ptr(), K + pad_x, y.data_ptr(), N + pad_y, M, capi.ACT_Q8, capi.KERNEL_AUTO), c.handle)
        c.sync()
        if world == 1 and M <= 4:
            dots = c.block_dots(h, xd[:, :K].contiguous())
            c.sync()
            assert (dots.cpu().numpy() == oracle.block_dots(w, x)).all()
        h.free()
        c.close()
    got = y.cpu().numpy()
    assert (got[:, N:] == -7.0).all()
    assert _rel(got[:, :N], ref) <= TOL, (case, N, K, M, world)


@pytest.mark.parametrize("case,N,K,M,seed", list(_cases(12, 777)))
def test_batches_norms_and_fused_tails_of_random_shapes(capi, oracle, case, N, K, M, seed):
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    K = max(K, 64) // 64 * 64
    rng = np.random.default_rng(seed)
    N2 = int(rng.integers(1, 1500))
    wa, wb = synth.make_weight(N, K, seed % 100003), synth.make_weight(N2, K, seed % 100019)
    x = synth.make_activation(M, K, seed % 99989)
    nw = rng.uniform(0.5, 1.5, K).astype(np.float32)
    c = capi.Context(0)
    c.use_torch_stream()
    ha, hb = c.upload(wa), c.upload(wb)
    xd, nwd = torch.from_numpy(x).cuda(), torch.from_numpy(nw).cuda()
    ya, yb = torch.zeros((M, N), device="cuda"), torch.zeros((M, N2), device="cuda")
    # two projections of one input in one call
    c.mul_mat_batch([(ha, xd, ya), (hb, xd, yb)])
    c.sync()
    assert _rel(ya.cpu().numpy(), oracle.mul_mat(po.Q8ACT_LANES, wa, x, threads=8)) <= TOL
    assert _rel(yb.cpu().numpy(), oracle.mul_mat(po.Q8ACT_LANES, wb, x, threads=8)) <= TOL
    # the same behind rms_norm x norm-weight
    c.rms_norm_mul_mat_batch([(ha, xd, ya), (hb, xd, yb)], nwd, 1e-5)
    c.sync()
    normed = oracle.rms_norm_mul(x, nw, float(np.float32(1e-5)), 0)
    assert _rel(ya.cpu().numpy(), oracle.mul_mat(po.Q8ACT_LANES, wa, normed, threads=8)) <= TOL
    assert _rel(yb.cpu().numpy(), oracle.mul_mat(po.Q8ACT_LANES, wb, normed, threads=8)) <= TOL
    # y = W (silu(gate) * up) + residual and y = W x + residual
    gate, up = (synth.make_activation(M, K, seed % 99971) * 2).astype(np.float32), synth.make_activation(M, K, seed % 99961)
    res = synth.make_activation(M, N, seed % 99929)
    gd, ud, rd = (torch.from_numpy(a).cuda() for a in (gate, up, res))
    y1 = c.mul_mat_swiglu_add(ha, gd, ud, rd)
    y2 = c.mul_mat_add(ha, xd, rd)
    c.sync()
    ref1 = oracle.add(oracle.mul_mat(po.Q8ACT_LANES, wa, oracle.swiglu(gate, up), threads=8), res)
    ref2 = oracle.add(oracle.mul_mat(po.Q8ACT_LANES, wa, x, threads=8), res)
    assert _rel(y1.cpu().numpy(), ref1) <= 3e-4  # expf on the two sides differs in the last bits
    assert _rel(y2.cpu().numpy(), ref2) <= TOL
    ha.free()
    hb.free()
    c.close()
