"""The CPU oracle against the reference's golden vectors and known-answer cases (no GPU)."""
import numpy as np
import pytest

from oracle import pyoracle as po


def _bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def test_fp16_all_codes_against_golden(oracle, golden):
    want = golden["fp16_codes_to_f32"]
    got = np.array([oracle.fp16_to_fp32(h) for h in range(65536)], dtype=np.float32).view(np.uint32)
    nan = (want & 0x7FFFFFFF) > 0x7F800000
    assert (got[~nan] == want[~nan]).all()
    assert ((got[nan] & 0x7FFFFFFF) > 0x7F800000).all()
    # and back: every non-NaN code survives a round trip
    for h in range(0, 65536, 1):
        if nan[h]:
            continue
        f = float(np.uint32(want[h]).view(np.float32))
        assert oracle.fp32_to_fp16(f) == h


def test_fp32_to_fp16_against_golden(oracle, golden):
    f = golden["fp16_in"]
    want = golden["fp16_out"]
    want_bt = golden["fp16_bittrick_out"]
    got = np.array([oracle.fp32_to_fp16(float(v)) for v in f], dtype=np.uint16)
    got_bt = np.array([oracle.fp32_to_fp16_bittrick(float(v)) for v in f], dtype=np.uint16)
    assert (got == want).all()
    assert (got_bt == want_bt).all()


def test_fp16_matches_numpy(oracle):
    rng = np.random.default_rng(3)
    f = np.concatenate([rng.standard_normal(2000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 3e4)])
    want = f.astype(np.float16).view(np.uint16)
    got = np.array([oracle.fp32_to_fp16(float(v)) for v in f], dtype=np.uint16)
    assert (got == want).all()


def test_quantiser_against_golden(oracle, golden):
    for i in range(len(golden["shapes"])):
        assert (oracle.quantize_rows(golden[f"w_f32_{i}"]) == golden[f"w_blocks_{i}"]).all()
        assert (oracle.quantize_rows(golden[f"x_f32_{i}"]) == golden[f"x_blocks_{i}"]).all()


@pytest.mark.parametrize("mode,key,exact", [(po.Q8ACT_LANES, "dot_lanes", True), (po.Q8ACT_CHUNK16, "dot_chunk16", True),
                                           (po.F32ACT_PROMPT, "dot_f32_prompt", True), (po.F32ACT_EVAL, "dot_f32_eval", False)])
def test_row_dots_against_golden(oracle, golden, mode, key, exact):
    for i, (rows, K) in enumerate(golden["shapes"]):
        w = golden[f"w_blocks_{i}"]
        want = golden[f"{key}_{i}"]
        got = np.zeros_like(want)
        for m in range(2):
            for n in range(rows):
                if mode in (po.Q8ACT_LANES, po.Q8ACT_CHUNK16):
                    got[m, n] = oracle.vec_dot_q8q8(mode, w[n], golden[f"x_blocks_{i}"][m])
                else:
                    got[m, n] = oracle.vec_dot_q8f32(mode, w[n], golden[f"x_f32_{i}"][m])
        if exact:
            assert (_bits(got) == _bits(want)).all(), (key, i)
        else:
            # the eval-time f32 variant rounds differently from compiler to compiler (see q8_oracle.c)
            assert np.abs(got - want).max() <= 1e-5 * max(np.abs(want).max(), 1e-30), (key, i)


def test_known_answers(oracle):
    # all-zero block: scale 0, quants 0
    z = oracle.quantize_rows(np.zeros((1, 32), np.float32))
    assert (z == 0).all()
    # saturating block: +-1 alternating -> d = fp16(1/127), q = +-127
    x = np.where(np.arange(32) % 2 == 0, 1.0, -1.0).astype(np.float32)[None, :]
    b = oracle.quantize_rows(x)[0, 0]
    assert b[:2].view(np.uint16)[0] == np.float16(1.0 / 127.0).view(np.uint16)
    assert (b[2:].view(np.int8) == np.where(np.arange(32) % 2 == 0, 127, -127)).all()
    # single spike
    x = np.zeros((1, 32), np.float32)
    x[0, 31] = -5.0
    b = oracle.quantize_rows(x)[0, 0]
    q = b[2:].view(np.int8)
    assert q[31] == -127 and (q[:31] == 0).all()
    # denormal fp16 scale: amax/127 below 6.1e-5
    x = np.full((1, 32), 1e-3, np.float32)
    b = oracle.quantize_rows(x)[0, 0]
    d = np.uint16(b[0] | (b[1] << 8)).view(np.float16)
    assert 0 < float(d) < 6.2e-5 and (b[2:].view(np.int8) == 127).all()
    # ties round to even: x*id = 0.5 -> 0, 1.5 -> 2, 2.5 -> 2
    x = np.zeros((1, 32), np.float32)
    x[0, 0] = 127.0
    x[0, 1:4] = [0.5, 1.5, 2.5]
    q = oracle.quantize_rows(x)[0, 0][2:].view(np.int8)
    assert list(q[:4]) == [127, 0, 2, 2]
    # dot of the saturating block with itself: 32 * 127 * 127 * d^2
    w = oracle.quantize_rows(np.where(np.arange(32) % 2 == 0, 1.0, -1.0).astype(np.float32)[None, :])
    d = float(np.float16(1.0 / 127.0))
    want = np.float32(32 * 127 * 127) * (np.float32(d) * np.float32(d))
    for mode in (po.Q8ACT_LANES, po.Q8ACT_SCALAR, po.Q8ACT_CHUNK16, po.Q8ACT_F64):
        assert oracle.vec_dot_q8q8(mode, w[0], w[0]) == pytest.approx(float(want), rel=1e-6)


def test_variants_agree_and_truth(oracle):
    """All orderings of the same products stay within 1e-4 of the fp64 accumulation (the parity tolerance)."""
    rng = np.random.default_rng(11)
    for N, K in ((64, 4096), (16, 14336), (33, 96)):
        w = oracle.quantize_rows((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
        x = rng.standard_normal((3, K)).astype(np.float32)
        truth = oracle.mul_mat(po.Q8ACT_F64, w, x)
        for mode in (po.Q8ACT_LANES, po.Q8ACT_SCALAR, po.Q8ACT_CHUNK16):
            y = oracle.mul_mat(mode, w, x)
            assert np.abs(y - truth).max() <= 1e-4 * np.abs(truth).max()
        truth = oracle.mul_mat(po.F32ACT_F64, w, x)
        for mode in (po.F32ACT_EVAL, po.F32ACT_PROMPT):
            y = oracle.mul_mat(mode, w, x)
            assert np.abs(y - truth).max() <= 1e-4 * np.abs(truth).max()


def test_block_dots_exact(oracle):
    rng = np.random.default_rng(5)
    w = oracle.quantize_rows((rng.standard_normal((7, 256)) * 0.02).astype(np.float32))
    x = rng.standard_normal((2, 256)).astype(np.float32)
    aq = oracle.quantize_rows(x)
    dots = oracle.block_dots(w, x)
    qw = w[:, :, 2:].view(np.int8).astype(np.int64)
    qa = aq[:, :, 2:].view(np.int8).astype(np.int64)
    want = np.einsum("nbj,mbj->mnb", qw, qa)
    assert (dots == want).all()


def test_mul_mat_layout_and_threads(oracle):
    rng = np.random.default_rng(6)
    w = oracle.quantize_rows((rng.standard_normal((37, 128)) * 0.02).astype(np.float32))
    x = rng.standard_normal((5, 128)).astype(np.float32)
    y1 = oracle.mul_mat(po.Q8ACT_LANES, w, x, threads=1)
    y4 = oracle.mul_mat(po.Q8ACT_LANES, w, x, threads=4)
    assert (_bits(y1) == _bits(y4)).all()
    aq = oracle.quantize_rows(x)
    for m in (0, 4):
        for n in (0, 36):
            assert y1[m, n] == np.float32(oracle.vec_dot_q8q8(po.Q8ACT_LANES, w[n], aq[m]))
    # row range: only [n0, n1) is written
    part = oracle.mul_mat(po.Q8ACT_LANES, w, x, n0=10, n1=20)
    assert (_bits(part[:, 10:20]) == _bits(y1[:, 10:20])).all() and (part[:, :10] == 0).all() and (part[:, 20:] == 0).all()
    # empty inputs
    assert oracle.mul_mat(po.Q8ACT_LANES, w, np.zeros((0, 128), np.float32)).shape == (0, 37)
    assert oracle.mul_mat(po.Q8ACT_LANES, w[:0], x).shape == (5, 0)


def test_repack_round_trip(oracle):
    rng = np.random.default_rng(8)
    w = oracle.quantize_rows((rng.standard_normal((19, 96)) * 0.02).astype(np.float32))
    q, d = oracle.repack(w, 3, 17)
    assert q.shape == (14, 96) and d.shape == (14, 3)
    assert (oracle.unpack(q, d) == w[3:17]).all()
    assert (q.reshape(14, 3, 32) == w[3:17, :, 2:].view(np.int8)).all()


def test_reference_in_place_build_matches_oracle(oracle, reference):
    """Where the reference tree was present at build time: its own compiled helpers, bit for bit."""
    if reference is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(21)
    for N, K in ((32, 4096), (8, 14336), (16, 64), (16, 1024)):
        wf = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        x = rng.standard_normal((2, K)).astype(np.float32)
        w = oracle.quantize_rows(wf)
        assert (w == reference.quantize_rows(wf)).all()
        assert (_bits(oracle.mul_mat(po.Q8ACT_LANES, w, x)) == _bits(reference.mul_mat(0, w, x))).all()
        assert (_bits(oracle.mul_mat(po.Q8ACT_CHUNK16, w, x)) == _bits(reference.mul_mat(2, w, x))).all()
        assert (_bits(oracle.mul_mat(po.F32ACT_PROMPT, w, x)) == _bits(reference.mul_mat(4, w, x))).all()
        yo, yr = oracle.mul_mat(po.F32ACT_EVAL, w, x), reference.mul_mat(3, w, x)
        assert np.abs(yo - yr).max() <= 1e-5 * np.abs(yr).max()


def test_synthetic_generator_matches_oracle_quantiser(oracle):
    from nihilus_b200 import synth

    rng = np.random.default_rng(2)
    x = (rng.standard_normal((40, 256)) * 0.02).astype(np.float32)
    x[0, :32] = 0
    x[1, :32] = 1e-30
    assert (synth.quantize_q8_0(x) == oracle.quantize_rows(x)).all()
    a = synth.make_weight(300, 128, 99, chunk_rows=64, threads=1)
    b = synth.make_weight(300, 128, 99, chunk_rows=64, threads=4)
    assert (a == b).all()
