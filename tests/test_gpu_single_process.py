"""One process, one host thread, several GPUs (needs at least two B200s): the way the reference's host would drive the
library (one process and one thread per model, cuda/thread_pool.hpp:46-67).

Every rank is a context of this process.  Outputs live in memory from nhb_symm_alloc_local (plain peer pointers, no IPC
handles, no NCCL); the decode GEMV delivers every rank's rows itself and launches wait for the peers where they read
delivered rows; the host enqueues every rank's work before it blocks (nhb_sync_all).  The prefill path completes its rows
with nhb_all_gather_local (peer copies ordered by events).  Results: the same bits on every rank and the bits of one GPU.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
def test_one_thread_drives_all_ranks(capi, oracle, world):
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    dims = [(14336, 4096), (4096, 14336), (1024, 4096)]
    ws = [synth.make_weight(n, k, 195 + i) for i, (n, k) in enumerate(dims)]
    x = synth.make_activation(1, 4096, 199)
    # one GPU, one context: the definition of the right answer
    solo = capi.Context(0)
    solo.use_torch_stream()
    hs1 = [solo.upload(w) for w in ws]
    v = torch.from_numpy(x).to("cuda:0")
    one_gpu = []
    for h in hs1:
        v = solo.mul_mat(h, v)
        one_gpu.append(v.cpu().numpy())
    solo.sync()
    assert np.abs(one_gpu[0] - oracle.mul_mat(po.Q8ACT_LANES, ws[0], x)).max() <= 1e-4 * np.abs(one_gpu[0]).max()
    for h in hs1:
        h.free()
    solo.close()

    ctxs = [capi.Context(d, d, world) for d in range(world)]
    try:
        for d, c in enumerate(ctxs):
            with torch.cuda.device(d):
                c.use_torch_stream()
            c.set_option("peer_wait_us", 500000)
        hs = [[c.upload(w) for w in ws] for c in ctxs]
        for d in range(world):
            assert (hs[d][0].n0, hs[d][0].n1) == capi.shard_rows(dims[0][0], world, d)
        xs = [torch.from_numpy(x).to(f"cuda:{d}") for d in range(world)]
        ys = [capi.symm_empty_local(ctxs, (1, n)) for n, _ in dims]  # ys[stage][rank]
        # ---- decode: three dependent sharded stages, ten rounds (every round rewrites what the round before read) ----
        for _ in range(10):
            for d, c in enumerate(ctxs):  # everything for rank d, then the next rank: nothing here blocks the host
                c.mul_mat(hs[d][0], xs[d], ys[0][d])
                c.mul_mat(hs[d][1], ys[0][d], ys[1][d])
                c.mul_mat(hs[d][2], ys[1][d], ys[2][d])
        capi.sync_all(ctxs)
        for i in range(3):
            for d in range(world):
                got = ys[i][d].cpu().numpy()
                assert (got.view(np.uint32) == one_gpu[i].view(np.uint32)).all(), (i, d)
        # ---- the same stages recorded as a chain per rank and captured into a graph per rank ----
        for t in ys[2]:
            t.zero_()
        for d in range(world):
            torch.cuda.synchronize(d)
        chains = [c.chain([[(hs[d][0], xs[d], ys[0][d])], [(hs[d][1], ys[0][d], ys[1][d])], [(hs[d][2], ys[1][d], ys[2][d])]]) for d, c in enumerate(ctxs)]
        for _ in range(3):
            for ch in chains:
                ch.launch()
        capi.sync_all(ctxs)
        for d in range(world):
            assert (ys[2][d].cpu().numpy().view(np.uint32) == one_gpu[2].view(np.uint32)).all(), d
        for ch in chains:
            ch.free()
        # ---- prefill: the GEMM writes each rank's columns, nhb_all_gather_local completes the rows ----
        M = 40
        xp = synth.make_activation(M, 4096, 201)
        ref = oracle.mul_mat(po.Q8ACT_LANES, ws[0], xp)
        xps = [torch.from_numpy(xp).to(f"cuda:{d}") for d in range(world)]
        yps = [torch.zeros((M, dims[0][0]), device=f"cuda:{d}") for d in range(world)]
        for d, c in enumerate(ctxs):
            c.mul_mat(hs[d][0], xps[d], yps[d])
        capi.all_gather_local(ctxs, yps)
        capi.sync_all(ctxs)
        first = yps[0].cpu().numpy()
        assert np.abs(first - ref).max() <= 1e-4 * np.abs(ref).max()
        for d in range(1, world):
            assert (yps[d].cpu().numpy().view(np.uint32) == first.view(np.uint32)).all(), d
        for row in hs:
            for h in row:
                h.free()
    finally:
        for c in ctxs:
            c.close()
