"""Row sharding + all-gather on CPU ranks (gloo, world_size 2 and 3): the host-side logic of the multi-GPU path."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, N, K, M, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nihilus_b200 import capi, synth
        from oracle import pyoracle as po

        oracle = po.Oracle()
        w = synth.make_weight(N, K, 77, threads=1)
        x = synth.make_activation(M, K, 78)
        n0, n1 = capi.shard_rows(N, world, rank)
        # what one rank owns: its rows of the repacked planes, and its output columns
        qp, dp = capi.repack_host(w, n0, n1)
        shard_blocks = capi.unpack_host(qp, dp)
        assert (shard_blocks == w[n0:n1]).all()
        y_part = oracle.mul_mat(po.Q8ACT_LANES, shard_blocks, x, threads=1)  # [M, n1-n0]
        # all-gather of ragged column slices -> [M, N] on every rank
        sizes = [capi.shard_rows(N, world, r) for r in range(world)]
        pad = max(b - a for a, b in sizes)
        send = torch.zeros((M, pad), dtype=torch.float32)
        send[:, : n1 - n0] = torch.from_numpy(y_part)
        recv = [torch.zeros((M, pad), dtype=torch.float32) for _ in range(world)]
        dist.all_gather(recv, send)
        y = np.concatenate([recv[r][:, : b - a].numpy() for r, (a, b) in enumerate(sizes)], axis=1)
        full = oracle.mul_mat(po.Q8ACT_LANES, w, x, threads=1)
        ok = bool((y.view(np.uint32) == full.view(np.uint32)).all())
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,N", [(2, 64), (3, 50)])
def test_sharded_rows_all_gather_equals_unsharded(world, N):
    from nihilus_b200 import build

    build.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000) + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, N, 256, 3, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = sorted(q.get(timeout=5) for _ in range(world))
    assert results == [(r, True) for r in range(world)]
