"""The bounded waits of the fused all-gather, on one GPU and without any fault (needs a B200).

A context that believes it is rank 0 of 2 gets "symmetric" memory whose peer mappings alias its own allocation
(option symm_loopback), so no other rank ever announces a launch.  Whoever then waits for the peers -- nhb_sync, or a
launch that reads the rows they were to deliver -- runs into its time limit, records a status word and carries on:
the kernel ends normally, nhb_sync reports NHB_ERR_TIMEOUT, and the context keeps working.  Nothing traps, nothing hangs.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_a_peer_that_never_announces_ends_in_a_timeout_status_not_a_hang(capi, oracle):
    import time

    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    N, K = 1024, 4096
    w = synth.make_weight(N, K, 11)
    x = synth.make_activation(1, K, 12)
    ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
    c = capi.Context(0, 0, 2)
    c.use_torch_stream()
    c.set_option("symm_loopback", 1)
    c.set_option("peer_wait_us", 3000)
    h = c.upload(w)
    assert (h.n0, h.n1) == (0, N // 2)
    xd = torch.from_numpy(x).cuda()
    y = c.symm_empty((1, N))
    c.mul_mat(h, xd, y)  # delivers its half and announces launch 1; nobody else ever will
    t0 = time.time()
    with pytest.raises(capi.NhbError) as e:
        c.sync()  # waits for the peers' announcement of launch 1, for 3 ms
    assert e.value.code == capi.ERR_TIMEOUT
    assert time.time() - t0 < 5.0
    got = y.cpu().numpy()
    assert np.abs(got[:, : N // 2] - ref[:, : N // 2]).max() <= 1e-4 * np.abs(ref).max()  # this rank's own columns are right
    assert (got[:, N // 2:] == 0).all()  # the peer's were never delivered
    c.sync()  # the status was cleared and the exchange reset: a second sync is clean
    # a GEMV launch that reads the rows the peer was to deliver runs into the same limit in its own prologue and still finishes
    w2 = synth.make_weight(512, N, 13)
    h2 = c.upload(w2)
    y2 = c.symm_empty((1, 512))
    c.mul_mat(h, xd, y)
    c.mul_mat(h2, y, y2)
    with pytest.raises(capi.NhbError) as e:
        c.sync()
    assert e.value.code == capi.ERR_TIMEOUT
    ref2 = oracle.mul_mat(po.Q8ACT_LANES, w2, y.cpu().numpy())
    assert np.abs(y2.cpu().numpy()[:, :256] - ref2[:, :256]).max() <= 1e-4 * np.abs(ref2).max()
    # with no window every launch keeps in step with the peers, whatever it reads: the limit is met in its prologue again
    c.set_option("peer_window", 0)
    y3 = c.symm_empty((1, N))
    c.mul_mat(h, xd, y)
    c.mul_mat(h, xd, y3)
    with pytest.raises(capi.NhbError) as e:
        c.sync()
    assert e.value.code == capi.ERR_TIMEOUT
    assert np.abs(y3.cpu().numpy()[:, : N // 2] - ref[:, : N // 2]).max() <= 1e-4 * np.abs(ref).max()
    h2.free()
    # the context is still good for work that needs no peer: a weight kept whole on every rank
    c.set_option("replicate_below_mb", 1000)
    hw = c.upload(w)
    assert (hw.n0, hw.n1) == (0, N)
    yw = torch.zeros((1, N), device="cuda")
    c.mul_mat(hw, xd, yw)
    c.sync()
    assert np.abs(yw.cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()
    h.free()
    hw.free()
    c.close()
