"""world_size-2 (and 3) gloo runs on CPU of the multi-GPU plumbing: token and column
sharding reproduce the single-process result exactly.  The per-rank arithmetic is the CPU
oracle here (on the GPU box it is the CUDA library); what is under test is the ranges, the
collectives and the re-layout."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, mode, M, K, N, v, CT, q):
    sys.path.insert(0, ROOT)
    import oracle
    import pim_dl_asplos_b200  # noqa: F401
    from pim_dl_asplos_b200 import shard, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = synth.make_case(M=M, K=K, N=N, v=v, CT=CT, seed=42)
        lut, bias = c.lut, c.bias
        if mode == "n":
            lut, bias = shard.shard_weights_by_columns(c.lut, c.bias, rank, world)
            lut, bias = np.ascontiguousarray(lut), np.ascontiguousarray(bias)

        def amm_fn(rows):
            if lut.shape[2] == 0 or rows.shape[0] == 0:
                return torch.zeros(rows.shape[0], lut.shape[2])
            out, _, _ = oracle.amm(np.ascontiguousarray(rows.numpy()), c.centroid, lut, bias, c.scale, nthreads=1)
            return torch.from_numpy(out)

        y = shard.run_sharded(amm_fn, torch.from_numpy(c.x), M, N, mode)
        want, _, _ = oracle.amm(c.x, c.centroid, c.lut, c.bias, c.scale, nthreads=1)
        q.put((rank, bool(np.array_equal(y.numpy().view(np.uint32), want.view(np.uint32))), tuple(y.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,mode,M,N", [(2, "m", 37, 64), (2, "n", 24, 96), (3, "m", 10, 32), (3, "n", 8, 64),
                                            (2, "n", 5, 16)])
def test_sharded_amm_equals_unsharded(world, mode, M, N):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 300) + world * 7 + (0 if mode == "m" else 1) + M
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, M, 32, N, 2, 8, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, shape in res:
        assert ok, f"rank {rank}: sharded result differs"
        assert shape == (M, N)


def test_ranges_partition_exactly():
    import pim_dl_asplos_b200  # noqa: F401
    from pim_dl_asplos_b200 import shard
    for M in (0, 1, 7, 12608, 65536):
        for world in (1, 2, 3, 4, 8):
            r = [shard.token_range(M, k, world) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == M
            assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
            assert max(hi - lo for lo, hi in r) - min(hi - lo for lo, hi in r) <= 1
    for N in (16, 768, 3072, 16384):
        for world in (1, 2, 4, 8):
            r = [shard.column_range(N, k, world) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == N
            assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
            assert all(lo % 16 == 0 and hi % 16 == 0 for lo, hi in r)
