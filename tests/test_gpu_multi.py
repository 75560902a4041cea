"""Row-sharded mul_mat on 2, 4 and 8 GPUs, one process per GPU: NCCL all-gather, the all-gather fused into the decode GEMV,
stage chains and the placement policy (each world size is skipped where the box has fewer devices)."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, uid_path, q):
    sys.path.insert(0, ROOT)
    import time

    import torch

    from nihilus_b200 import capi, synth

    torch.cuda.set_device(rank)
    ctx = capi.Context(rank, rank, world)
    ctx.use_torch_stream()
    # rank 0 makes the NCCL id; the others pick it up from a file (any transport will do)
    if rank == 0:
        uid = capi.Context.comm_unique_id()
        with open(uid_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(uid_path + ".tmp", uid_path)
    else:
        for _ in range(600):
            if os.path.exists(uid_path):
                break
            time.sleep(0.05)
        uid = open(uid_path, "rb").read()
    ctx.comm_init(uid)
    out = {}
    for name, (N, K, M) in {"even": (4096, 4096, 1), "ragged": (1031, 4096, 3), "qkv": (1024, 4096, 2)}.items():
        w = synth.make_weight(N, K, 900 + N)
        x = torch.from_numpy(synth.make_activation(M, K, 901 + N)).cuda()
        h = ctx.upload(w)
        y = torch.zeros((M, N), device="cuda")
        ctx.mul_mat(h, x, y)
        ctx.all_gather(y)
        ctx.sync()
        out[name] = y.cpu().numpy()
        h.free()
    # two outputs in one grouped collective
    wa, wb = synth.make_weight(512, 4096, 77), synth.make_weight(256, 4096, 78)
    x = torch.from_numpy(synth.make_activation(1, 4096, 79)).cuda()
    ha, hb = ctx.upload(wa), ctx.upload(wb)
    ya, yb = torch.zeros((1, 512), device="cuda"), torch.zeros((1, 256), device="cuda")
    ctx.mul_mat_batch([(ha, x, ya), (hb, x, yb)])
    ctx.all_gather_batch([ya, yb])
    ctx.sync()
    out["batch_a"], out["batch_b"] = ya.cpu().numpy(), yb.cpu().numpy()
    # ---- fused all-gather: outputs in symmetric memory, the GEMV itself delivers every rank's columns ----
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ctx.use_torch_stream()
        cases = {"f_even": (4096, 4096, 1), "f_ragged": (1031, 4096, 3), "f_m8": (300, 512, 8)}
        ys, hs, xs = {}, {}, {}
        for name, (N, K, M) in cases.items():  # same allocations, same order, on every rank
            ys[name] = ctx.symm_empty((M, N))
        yq, yk = ctx.symm_empty((1, 512)), ctx.symm_empty((1, 256))
        for name, (N, K, M) in cases.items():
            hs[name] = ctx.upload(synth.make_weight(N, K, 900 + N))
            xs[name] = torch.from_numpy(synth.make_activation(M, K, 901 + N)).cuda()
        launches0 = ctx.launches
        for rep in range(3):  # repeated launches walk the epoch counter
            for name in cases:
                ctx.mul_mat(hs[name], xs[name], ys[name])
                ctx.all_gather(ys[name])  # nothing left to do: no collective is enqueued
            ctx.mul_mat_batch([(ha, x, yq), (hb, x, yk)])
            ctx.all_gather_batch([yq, yk])
        ctx.sync()
        out["fused_launches_per_rep"] = (ctx.launches - launches0) / 3
        for name in cases:
            out[name] = ys[name].cpu().numpy()
        out["f_batch_a"], out["f_batch_b"] = yq.cpu().numpy(), yk.cpu().numpy()
        # the same sequence replayed from a CUDA graph
        for name in cases:
            ys[name].zero_()
        ctx.sync()
        ctx.graph_begin()
        for name in cases:
            ctx.mul_mat(hs[name], xs[name], ys[name])
        g = ctx.graph_end()
        g.launch()
        g.launch()
        ctx.sync()
        for name in cases:
            out["g_" + name[2:]] = ys[name].cpu().numpy()
        g.free()
        for h in hs.values():
            h.free()
        # ---- rms_norm x norm-weight fused in front of a sharded stage whose outputs the GEMV delivers to every rank ----
        wn_a, wn_b = synth.make_weight(4096, 4096, 81), synth.make_weight(1024, 4096, 82)
        hn_a, hn_b = ctx.upload(wn_a), ctx.upload(wn_b)
        xn = torch.from_numpy(synth.make_activation(1, 4096, 83) * 2.0).cuda()
        nw = torch.from_numpy(np.linspace(0.5, 1.5, 4096, dtype=np.float32)).cuda()
        yn_a, yn_b = ctx.symm_empty((1, 4096)), ctx.symm_empty((1, 1024))
        for _ in range(2):
            ctx.rms_norm_mul_mat_batch([(hn_a, xn, yn_a), (hn_b, xn, yn_b)], nw, 1e-5)
            ctx.all_gather_batch([yn_a, yn_b])
        ctx.sync()
        out["n_a"], out["n_b"] = yn_a.cpu().numpy(), yn_b.cpu().numpy()
        hn_a.free()
        hn_b.free()
        # ---- placement policy: small weights stay whole on every rank, large ones are sharded; one batch mixes both ----
        ctx.set_option("replicate_below_mb", 4)
        w_small, w_big = synth.make_weight(700, 4096, 61), synth.make_weight(2048, 4096, 62)  # 3.0 MB and 8.9 MB
        hs_small, hs_big = ctx.upload(w_small), ctx.upload(w_big)
        out["small_rows"] = (hs_small.n0, hs_small.n1)
        out["big_rows"] = (hs_big.n0, hs_big.n1)
        xr = torch.from_numpy(synth.make_activation(2, 4096, 63)).cuda()
        ys_small, ys_big = ctx.symm_empty((2, 700)), ctx.symm_empty((2, 2048))
        l0 = ctx.launches
        for _ in range(2):
            ctx.mul_mat_batch([(hs_small, xr, ys_small), (hs_big, xr, ys_big)])
            ctx.all_gather_batch([ys_small, ys_big])
            ctx.mul_mat(hs_small, xr, ys_small)  # all ops replicated: no exchange at all
            ctx.all_gather(ys_small)
        ctx.sync()
        out["policy_launches"] = ctx.launches - l0
        out["p_small"], out["p_big"] = ys_small.cpu().numpy(), ys_big.cpu().numpy()
        hs_small.free()
        hs_big.free()
        ctx.set_option("replicate_below_mb", 0)
        # ---- a buffer written again two delivering launches later, with a reader in between (the documented reuse rule) ----
        wp = synth.make_weight(2048, 4096, 91)
        hp = ctx.upload(wp)
        bufs = [ctx.symm_empty((1, 2048)), ctx.symm_empty((1, 2048))]
        xp = [torch.from_numpy(synth.make_activation(1, 4096, 92 + j)).cuda() for j in range(6)]
        logs = [torch.zeros((1, 2048), device="cuda") for _ in range(6)]
        for j in range(6):
            ctx.mul_mat(hp, xp[j], bufs[j % 2])
            ctx.all_gather(bufs[j % 2])  # the reader below is not a GEMV launch: this is where it waits for the peers
            logs[j].copy_(bufs[j % 2])
        ctx.sync()
        out["pingpong"] = [t.cpu().numpy() for t in logs]
        # ---- a chain of dependent stages: 4096 -> 14336 -> 4096 -> 1024, every stage sharded and delivered ----
        dims = [(14336, 4096), (4096, 14336), (1024, 4096)]
        hc = [ctx.upload(synth.make_weight(n, k, 95 + i)) for i, (n, k) in enumerate(dims)]
        xc = torch.from_numpy(synth.make_activation(1, 4096, 99)).cuda()
        yc = [ctx.symm_empty((1, n)) for n, _ in dims]
        ch = ctx.chain([[(hc[0], xc, yc[0])], [(hc[1], yc[0], yc[1])], [(hc[2], yc[1], yc[2])]])
        for rnd in range(10):  # every round rewrites what the round before read: the launches wait for exactly that
            if rnd == 4 and rank == world - 1:
                time.sleep(0.3)  # a rank that is late by less than the waits' limit (2 s): the others wait for it on the device
            ch.launch()
        ctx.all_gather(yc[2])
        ctx.sync()
        out["chain"] = [t.cpu().numpy() for t in yc]
        ch.free()
        for h in hc + [hp]:
            h.free()
    q.put((rank, out))
    ha.free()
    hb.free()
    ctx.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shards_delivered_to_every_rank_match_oracle_and_one_gpu(capi, oracle, tmp_path, world):
    import torch
    import torch.multiprocessing as mp

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mpctx = mp.get_context("spawn")
    q = mpctx.Queue()
    uid_path = str(tmp_path / "nccl_uid.bin")
    procs = [mpctx.Process(target=_worker, args=(r, world, uid_path, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    ranks = range(world)

    def same_on_all_ranks(key):
        for r in ranks:
            assert (np.asarray(results[r][key]).view(np.uint32) == np.asarray(results[0][key]).view(np.uint32)).all(), (key, r)

    def close(y, ref):
        return np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()

    for name, (N, K, M) in {"even": (4096, 4096, 1), "ragged": (1031, 4096, 3), "qkv": (1024, 4096, 2)}.items():
        ref = oracle.mul_mat(po.Q8ACT_LANES, synth.make_weight(N, K, 900 + N), synth.make_activation(M, K, 901 + N))
        for r in ranks:
            assert close(results[r][name], ref), (name, r)
        same_on_all_ranks(name)
    x = synth.make_activation(1, 4096, 79)
    for key, seed, N in (("batch_a", 77, 512), ("batch_b", 78, 256)):
        ref = oracle.mul_mat(po.Q8ACT_LANES, synth.make_weight(N, 4096, seed), x)
        for r in ranks:
            assert close(results[r][key], ref)
            # fused delivery gives the very same bits as compute + NCCL
            assert (results[r]["f_" + key].view(np.uint32) == results[r][key].view(np.uint32)).all()
    for name, (N, K, M) in {"even": (4096, 4096, 1), "ragged": (1031, 4096, 3), "m8": (300, 512, 8)}.items():
        ref = oracle.mul_mat(po.Q8ACT_LANES, synth.make_weight(N, K, 900 + N), synth.make_activation(M, K, 901 + N))
        for r in ranks:
            for prefix in ("f_", "g_"):
                assert close(results[r][prefix + name], ref), (prefix, name, r)
            assert (results[r]["f_" + name].view(np.uint32) == results[0]["g_" + name].view(np.uint32)).all()
        if name in ("even", "ragged"):
            assert (results[0]["f_" + name].view(np.uint32) == results[0][name].view(np.uint32)).all()
    normed = oracle.rms_norm_mul((synth.make_activation(1, 4096, 83) * 2.0).astype(np.float32), np.linspace(0.5, 1.5, 4096, dtype=np.float32),
                                 float(np.float32(1e-5)), 0)
    for key, seed, N in (("n_a", 81, 4096), ("n_b", 82, 1024)):
        ref = oracle.mul_mat(po.Q8ACT_LANES, synth.make_weight(N, 4096, seed), normed)
        for r in ranks:
            assert close(results[r][key], ref), (key, r)
        same_on_all_ranks(key)
    xr = synth.make_activation(2, 4096, 63)
    for key, seed, N in (("p_small", 61, 700), ("p_big", 62, 2048)):
        ref = oracle.mul_mat(po.Q8ACT_LANES, synth.make_weight(N, 4096, seed), xr)
        for r in ranks:
            assert close(results[r][key], ref), (key, r)
        same_on_all_ranks(key)
    for r in ranks:
        assert results[r]["small_rows"] == (0, 700)  # whole on every rank
        assert results[r]["big_rows"] == capi.shard_rows(2048, world, r)
        # per repetition: the mixed batch, the wait for its delivery, the replicated-only launch; never a collective
        assert results[r]["policy_launches"] == 6
    # per repetition 3 single mul_mats (8 rows go in one pass) + 1 batch, each followed by a one-warp wait; no NCCL launch
    assert results[0]["fused_launches_per_rep"] == 8
    # buffers reused every second delivering launch, a reader in between: every reader saw its own launch's rows, whole
    wp = synth.make_weight(2048, 4096, 91)
    for j in range(6):
        ref = oracle.mul_mat(po.Q8ACT_LANES, wp, synth.make_activation(1, 4096, 92 + j))
        for r in ranks:
            assert close(results[r]["pingpong"][j], ref), (j, r)
    # the chain: bit-identical on all ranks and to the same chain on ONE GPU (the definition of parity for the sharded path)
    c1 = capi.Context(0)
    c1.use_torch_stream()
    dims = [(14336, 4096), (4096, 14336), (1024, 4096)]
    ws = [synth.make_weight(n, k, 95 + i) for i, (n, k) in enumerate(dims)]
    hs = [c1.upload(w) for w in ws]
    v = torch.from_numpy(synth.make_activation(1, 4096, 99)).cuda()
    one_gpu = []
    for h in hs:
        v = c1.mul_mat(h, v)
        one_gpu.append(v)
    c1.sync()
    for i in range(3):
        for r in ranks:
            assert (results[r]["chain"][i].view(np.uint32) == one_gpu[i].cpu().numpy().view(np.uint32)).all(), (i, r)
    assert close(one_gpu[0].cpu().numpy(), oracle.mul_mat(po.Q8ACT_LANES, ws[0], synth.make_activation(1, 4096, 99)))
    for h in hs:
        h.free()
    c1.close()
