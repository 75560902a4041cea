"""SwiGLU and residual-add fused into the decode GEMV (and run around the GEMM for prefill) against the separate steps and
the CPU oracle (needs a B200).  Reference chains: ffn_gate_mul_mat -> silu -> mul(ffn_up_mul_mat) -> ffn_down_mul_mat ->
add(ffn_inp) and attn_out_mul_mat -> add(inp_embd) (include/nihilus-incl/infra/core_traits.hpp:768-772, 976-992)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-4  # max|err| / max|ref| of a mul_mat output
SWIGLU_TOL = 2e-6  # silu(g) * u against the oracle: the two exp() implementations differ in the last bits


def _rel(y, ref):
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.fixture(scope="module")
def ctx(capi):
    c = capi.Context(0)
    c.use_torch_stream()
    yield c
    c.close()


def test_oracle_swiglu_agrees_with_its_fp64_form(oracle):
    rng = np.random.default_rng(3)
    g = (rng.standard_normal(100000) * 3).astype(np.float32)
    u = rng.standard_normal(100000).astype(np.float32)
    g[:6] = [0.0, -0.0, 50.0, -50.0, 88.0, -88.0]
    a, b = oracle.swiglu(g, u), oracle.swiglu(g, u, f64=True)
    assert np.isfinite(a).all()
    assert np.abs(a - b).max() <= 2e-7 * np.abs(b).max()
    assert (oracle.add(g, u) == g + u).all()


@pytest.mark.parametrize("M", [1, 3, 4, 7, 40])
def test_ffn_tail_fused_equals_the_separate_steps_and_the_oracle(capi, ctx, oracle, M):
    """gate/up rows -> SwiGLU -> quantise -> ffn_down -> + residual, in one call: the bits of nhb_swiglu + nhb_mul_mat + add."""
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    FF, E = 14336, 1024  # ffn_down's K at full size (the long-row kernels), fewer rows to keep the oracle quick
    w = synth.make_weight(E, FF, 4100)
    h = ctx.upload(w)
    gate = (synth.make_activation(M, FF, 4101 + M) * 2).astype(np.float32)
    up = synth.make_activation(M, FF, 4102 + M)
    res = synth.make_activation(M, E, 4103 + M)
    gd, ud, rd = (torch.from_numpy(a).cuda() for a in (gate, up, res))
    hd = ctx.swiglu(gd, ud)
    ctx.sync()
    ref_h = oracle.swiglu(gate, up)
    assert _rel(hd.cpu().numpy(), ref_h) <= SWIGLU_TOL
    assert _rel(hd.cpu().numpy(), oracle.swiglu(gate, up, f64=True)) <= SWIGLU_TOL
    two_step = ctx.mul_mat(h, hd) + rd
    fused = ctx.mul_mat_swiglu_add(h, gd, ud, rd)
    no_res = ctx.mul_mat_swiglu_add(h, gd, ud)
    ctx.sync()
    assert torch.equal(fused, two_step)
    assert torch.equal(no_res, ctx.mul_mat(h, hd))
    # the oracle's chain from the GPU's own SwiGLU rows (so that a last-bit difference in exp() cannot flip a quantised activation) ...
    ref = oracle.add(oracle.mul_mat(po.Q8ACT_LANES, w, hd.cpu().numpy()), res)
    assert _rel(fused.cpu().numpy(), ref) <= TOL
    # ... and end to end from the oracle's SwiGLU rows
    ref2 = oracle.add(oracle.mul_mat(po.Q8ACT_LANES, w, ref_h), res)
    assert _rel(fused.cpu().numpy(), ref2) <= 3 * TOL
    h.free()


@pytest.mark.parametrize("N,K,M", [(4096, 4096, 1), (1031, 4096, 3), (300, 512, 2), (4096, 4096, 20)])
def test_attention_output_with_the_residual_added_as_rows_are_stored(capi, ctx, oracle, N, K, M):
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    w = synth.make_weight(N, K, 4200 + N)
    h = ctx.upload(w)
    x = synth.make_activation(M, K, 4201 + M)
    res = synth.make_activation(M, N, 4202 + M)
    xd = torch.from_numpy(x).cuda()
    rd = torch.full((M, N + 4), 9.0, device="cuda")  # a residual with its own leading dimension
    rd[:, :N] = torch.from_numpy(res).cuda()
    y = torch.full((M, N + 2), -5.0, device="cuda")
    capi._check(capi.lib.nhb_mul_mat_add(ctx.handle, h.handle, xd.data_ptr(), K, rd.data_ptr(), N + 4, y.data_ptr(), N + 2, M), ctx.handle)
    want = ctx.mul_mat(h, xd) + rd[:, :N]
    ctx.sync()
    assert torch.equal(y[:, :N], want)
    assert (y[:, N:] == -5.0).all()
    assert _rel(y[:, :N].cpu().numpy(), oracle.add(oracle.mul_mat(po.Q8ACT_LANES, w, x), res)) <= TOL
    h.free()


def test_row_shards_of_the_fused_tail_are_bit_identical_to_one_gpu(capi, ctx):
    import torch

    from nihilus_b200 import synth

    FF, E, M = 14336, 1030, 2
    w = synth.make_weight(E, FF, 4300)
    gd = torch.from_numpy(synth.make_activation(M, FF, 4301)).cuda()
    ud = torch.from_numpy(synth.make_activation(M, FF, 4302)).cuda()
    rd = torch.from_numpy(synth.make_activation(M, E, 4303)).cuda()
    h = ctx.upload(w)
    full = ctx.mul_mat_swiglu_add(h, gd, ud, rd)
    ctx.sync()
    h.free()
    for world in (2, 3):
        y = torch.zeros((M, E), device="cuda")
        for r in range(world):
            c = capi.Context(0, r, world)
            c.use_torch_stream()
            hr = c.upload(w)
            c.mul_mat_swiglu_add(hr, gd, ud, rd, y=y)
            c.sync()
            hr.free()
            c.close()
        assert torch.equal(y, full)


def test_argument_errors(capi, ctx):
    import torch

    from nihilus_b200 import synth

    h = ctx.upload(synth.make_weight(64, 256, 1))
    g = torch.zeros((1, 256), device="cuda")
    y = torch.zeros((1, 64), device="cuda")
    lib = capi.lib
    assert lib.nhb_mul_mat_swiglu_add(ctx.handle, h.handle, g.data_ptr(), None, 256, None, 64, y.data_ptr(), 64, 1) == capi.ERR_ARG
    assert lib.nhb_mul_mat_add(ctx.handle, h.handle, g.data_ptr(), 256, None, 64, y.data_ptr(), 64, 1) == capi.ERR_ARG
    assert lib.nhb_mul_mat_add(ctx.handle, h.handle, g.data_ptr(), 256, y.data_ptr(), 32, y.data_ptr(), 64, 1) == capi.ERR_ARG  # ld_residual < N
    assert lib.nhb_swiglu(ctx.handle, g.data_ptr(), g.data_ptr(), 256, y.data_ptr(), 64, 1, 256) == capi.ERR_ARG  # ldh < K
    ctx.sync()
    h.free()
