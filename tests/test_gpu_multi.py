"""Row-sharded mul_mat + NCCL all-gather on 2 GPUs, one process per GPU (skipped with fewer than 2 devices)."""
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
    q.put((rank, out))
    ha.free()
    hb.free()
    ctx.close()


def test_two_gpu_shards_all_gathered_match_oracle(capi, oracle, tmp_path):
    import torch
    import torch.multiprocessing as mp

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mpctx = mp.get_context("spawn")
    q = mpctx.Queue()
    uid_path = str(tmp_path / "nccl_uid.bin")
    procs = [mpctx.Process(target=_worker, args=(r, world, uid_path, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for name, (N, K, M) in {"even": (4096, 4096, 1), "ragged": (1031, 4096, 3), "qkv": (1024, 4096, 2)}.items():
        w = synth.make_weight(N, K, 900 + N)
        x = synth.make_activation(M, K, 901 + N)
        ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
        for r in range(world):
            y = results[r][name]
            assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max(), (name, r)
        assert (results[0][name].view(np.uint32) == results[1][name].view(np.uint32)).all()
    x = synth.make_activation(1, 4096, 79)
    for key, seed, N in (("batch_a", 77, 512), ("batch_b", 78, 256)):
        ref = oracle.mul_mat(po.Q8ACT_LANES, synth.make_weight(N, 4096, seed), x)
        for r in range(world):
            assert np.abs(results[r][key] - ref).max() <= 1e-4 * np.abs(ref).max()
            # fused delivery gives the very same bits as compute + NCCL
            assert (results[r]["f_" + key].view(np.uint32) == results[r][key].view(np.uint32)).all()
    for name, (N, K, M) in {"even": (4096, 4096, 1), "ragged": (1031, 4096, 3), "m8": (300, 512, 8)}.items():
        ref = oracle.mul_mat(po.Q8ACT_LANES, synth.make_weight(N, K, 900 + N), synth.make_activation(M, K, 901 + N))
        for r in range(world):
            for prefix in ("f_", "g_"):
                y = results[r][prefix + name]
                assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max(), (prefix, name, r)
            assert (results[r]["f_" + name].view(np.uint32) == results[0]["g_" + name].view(np.uint32)).all()
        if name in ("even", "ragged"):
            assert (results[0]["f_" + name].view(np.uint32) == results[0][name].view(np.uint32)).all()
    normed = oracle.rms_norm_mul((synth.make_activation(1, 4096, 83) * 2.0).astype(np.float32), np.linspace(0.5, 1.5, 4096, dtype=np.float32),
                                 float(np.float32(1e-5)), 0)
    for key, seed, N in (("n_a", 81, 4096), ("n_b", 82, 1024)):
        ref = oracle.mul_mat(po.Q8ACT_LANES, synth.make_weight(N, 4096, seed), normed)
        for r in range(world):
            assert np.abs(results[r][key] - ref).max() <= 1e-4 * np.abs(ref).max(), (key, r)
        assert (results[0][key].view(np.uint32) == results[1][key].view(np.uint32)).all()
    xr = synth.make_activation(2, 4096, 63)
    for key, seed, N in (("p_small", 61, 700), ("p_big", 62, 2048)):
        ref = oracle.mul_mat(po.Q8ACT_LANES, synth.make_weight(N, 4096, seed), xr)
        for r in range(world):
            assert np.abs(results[r][key] - ref).max() <= 1e-4 * np.abs(ref).max(), (key, r)
        assert (results[0][key].view(np.uint32) == results[1][key].view(np.uint32)).all()
    for r in range(world):
        assert results[r]["small_rows"] == (0, 700)  # whole on every rank
        assert results[r]["big_rows"] == ((0, 1024), (1024, 2048))[r]
        assert results[r]["policy_launches"] == 4  # two kernels per repetition, never a collective
    # 3 single mul_mats (8 rows go in one pass) + 1 batch per repetition, and no NCCL launch at all
    assert results[0]["fused_launches_per_rep"] == 4
