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
