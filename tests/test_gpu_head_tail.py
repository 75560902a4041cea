"""The Q8_0 consumers on either side of the projections -- token-embedding gather, final norm + logits -- and the cache of
repacked weights (needs a B200)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-4


def _rel(y, ref):
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.fixture(scope="module")
def ctx(capi):
    c = capi.Context(0)
    c.use_torch_stream()
    yield c
    c.close()


def test_embedding_gather_is_bit_exact_and_honours_the_token_id(capi, ctx, oracle):
    """cuda/cuda_12.hpp:560-601: scale * float(q), one row per token.  Repeated ids, the first and the last row, a ragged
    output leading dimension; the products are exact in f32, so the comparison is bit for bit."""
    import torch

    from nihilus_b200 import synth

    V, E = 5000, 4096
    table = synth.make_weight(V, E, 6100)
    h = ctx.upload(table)
    ids = np.array([0, V - 1, 17, 17, 4242, 1, 0], dtype=np.int32)
    y = torch.full((ids.size, E + 8), -2.0, device="cuda")
    capi._check(capi.lib.nhb_get_rows_q8_0(ctx.handle, h.handle, torch.from_numpy(ids).cuda().data_ptr(), ids.size, y.data_ptr(), E + 8), ctx.handle)
    ctx.sync()
    got = y.cpu().numpy()
    ref = oracle.get_rows(table, ids)
    assert (got[:, :E].view(np.uint32) == ref.view(np.uint32)).all()
    assert (got[:, E:] == -2.0).all()
    assert not (ref[0] == ref[2]).all()  # different tokens, different rows: the id is honoured
    # one token (the decode phase) goes through the same kernel
    one = ctx.get_rows(h, torch.tensor([4242], dtype=torch.int32, device="cuda"))
    ctx.sync()
    assert (one.cpu().numpy().view(np.uint32) == ref[4:5].view(np.uint32)).all()
    # an id outside the table: reported, its row untouched, nothing faults
    bad = torch.full((2, E), 7.0, device="cuda")
    ctx.get_rows(h, torch.tensor([3, V], dtype=torch.int32, device="cuda"), y=bad)
    with pytest.raises(capi.NhbError) as e:
        ctx.sync()
    assert e.value.code == capi.ERR_ARG and "token id" in str(e.value)
    out = bad.cpu().numpy()
    assert (out[0].view(np.uint32) == oracle.get_rows(table, np.array([3], dtype=np.int32))[0].view(np.uint32)).all() and (out[1] == 7.0).all()
    ctx.sync()
    h.free()


def test_gather_needs_the_whole_table(capi):
    import torch

    from nihilus_b200 import synth

    c = capi.Context(0, 0, 2)
    c.use_torch_stream()
    h = c.upload(synth.make_weight(64, 256, 1))  # sharded: rank 0 of 2 holds half the rows
    y = torch.zeros((1, 256), device="cuda")
    ids = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert capi.lib.nhb_get_rows_q8_0(c.handle, h.handle, ids.data_ptr(), 1, y.data_ptr(), 256) == capi.ERR_UNSUPPORTED
    c.set_option("replicate_below_mb", 1)
    h2 = c.upload(synth.make_weight(64, 256, 1))
    assert capi.lib.nhb_get_rows_q8_0(c.handle, h2.handle, ids.data_ptr(), 1, y.data_ptr(), 256) == 0
    c.sync()
    h.free()
    h2.free()
    c.close()


@pytest.mark.parametrize("seq", [1, 5])
def test_last_token_logits_against_the_oracle(capi, ctx, oracle, seq):
    """infra/core_traits.hpp:1184-1193: view of the last token -> rms_norm -> x output_norm -> logits mul_mat."""
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    V, E = 6000, 4096
    w = synth.make_weight(V, E, 6200)
    h = ctx.upload(w)
    hidden = (synth.make_activation(seq, E, 6201 + seq) * 3).astype(np.float32)
    nw = np.linspace(0.5, 1.5, E, dtype=np.float32)
    hd, nwd = torch.from_numpy(hidden).cuda(), torch.from_numpy(nw).cuda()
    logits = ctx.last_token_logits(h, hd, nwd, 1e-5)
    # the same through the two separate calls: bit for bit
    normed = ctx.rms_norm_mul(hd[seq - 1:seq], nwd, 1e-5)
    two = ctx.mul_mat(h, normed)
    ctx.sync()
    assert torch.equal(logits, two)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w, oracle.rms_norm_mul(hidden[seq - 1:seq], nw, float(np.float32(1e-5)), 0))
    assert _rel(logits.cpu().numpy(), ref) <= TOL
    h.free()


def test_weight_cache_round_trip_and_refusals(capi, ctx, oracle, tmp_path):
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    N, K = 1031, 4096
    w = synth.make_weight(N, K, 6300)
    h = ctx.upload(w)
    path = str(tmp_path / "w.nhbw")
    h.save(path)
    back = ctx.load_weight(path, N, K)
    assert (back.n0, back.n1, back.N, back.K, back.bytes_q8) == (h.n0, h.n1, N, K, h.bytes_q8)
    assert (back.download() == w).all()
    x = torch.from_numpy(synth.make_activation(2, K, 6301)).cuda()
    ya, yb = ctx.mul_mat(h, x), ctx.mul_mat(back, x)
    ctx.sync()
    assert torch.equal(ya, yb)
    assert _rel(yb.cpu().numpy(), oracle.mul_mat(po.Q8ACT_LANES, w, x.cpu().numpy())) <= TOL
    # wrong shape, another rank's shard, a damaged file
    for args in ((N + 1, K), (N, K // 2)):
        with pytest.raises(capi.NhbError):
            ctx.load_weight(path, *args)
    c2 = capi.Context(0, 1, 2)
    c2.use_torch_stream()
    with pytest.raises(capi.NhbError, match="needs rows"):
        c2.load_weight(path, N, K)
    h2 = c2.upload(w)
    p2 = str(tmp_path / "shard.nhbw")
    h2.save(p2)
    b2 = c2.load_weight(p2, N, K)
    assert (b2.n0, b2.n1) == capi.shard_rows(N, 2, 1) and (b2.download() == w[b2.n0:b2.n1]).all()
    with pytest.raises(capi.NhbError, match="needs rows"):
        ctx.load_weight(p2, N, K)  # a shard file offered to the one-GPU context
    data = bytearray(open(path, "rb").read())
    data[200] ^= 0x55
    bad = str(tmp_path / "bad.nhbw")
    open(bad, "wb").write(bytes(data))
    with pytest.raises(capi.NhbError, match="checksum"):
        ctx.load_weight(bad, N, K)
    open(bad, "wb").write(bytes(data[:1000]))
    with pytest.raises(capi.NhbError, match="truncated"):
        ctx.load_weight(bad, N, K)
    open(bad, "wb").write(b"not a cache file at all, just some bytes that are long enough to hold a header ............................")
    with pytest.raises(capi.NhbError, match="not a weight cache"):
        ctx.load_weight(bad, N, K)
    for hh in (h, back, h2, b2):
        hh.free()
    c2.close()
