"""One rank of the sharded-operator GPU test (launched by tests/test_shard_gpu.py through torchrun).

Each rank: joins the library's own NCCL communicator, runs the column-sharded AMM (both search modes) and
the token-sharded AMM (with and without the row all-gather) through the C ABI, and compares every result
with the CPU oracle's unsharded output bit for bit.  NVLS is switched off by the launcher: the test only
needs plain peer transfers.  Exit code 0 = every comparison held on this rank.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np
import torch
import torch.distributed as dist

import oracle
import pim_dl_asplos_b200 as P
from pim_dl_asplos_b200 import shard, synth


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = P.LutAmmContext(local)
    ctx.shard_init()
    M, K, N, v, CT = 512 * world, 256, 384 * world, 2, 16
    c = synth.make_case(M=M, K=K, N=N, v=v, CT=CT, seed=3)
    want = oracle.amm(c.x, c.centroid, c.lut, c.bias, c.scale, 0.0)[0]
    x = torch.from_numpy(c.x).cuda()
    n_loc = N // world
    # ---- columns: this rank's slab of table and bias
    lo, hi = shard.column_range(N, rank, world)
    assert hi - lo == n_loc
    ctx.load_weights(0, c.centroid, np.ascontiguousarray(c.lut[:, :, lo:hi]), np.ascontiguousarray(c.bias[lo:hi]), c.scale)
    for plan in (dict(variant=P.VARIANT_AUTO), dict(variant=P.VARIANT_GATHER)):
        ctx.set_plan(0, **plan)
        for mode in (P.SHARD_SEARCH_REPLICATED, P.SHARD_SEARCH_SPLIT):
            gathered = torch.full((world, M, n_loc), float("nan"), device="cuda")
            ctx.amm_column_sharded(0, x, gathered, n_tokens=M, search_mode=mode)
            got = gathered.permute(1, 0, 2).reshape(M, N).cpu().numpy()
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (rank, plan, mode, "column-sharded")
            # the gathered buffer is the reference's tiled layout for lut_parallelism = world
            offs = np.array([oracle.tiled_output_offset(i, j, M, n_loc, n_loc, world) for i in (0, M - 1) for j in (0, n_loc, N - 1)])
            flat = gathered.reshape(-1).cpu().numpy()
            ref = np.array([want[i, j] for i in (0, M - 1) for j in (0, n_loc, N - 1)])
            assert np.array_equal(flat[offs].view(np.uint32), ref.view(np.uint32)), "not the reference's tiled layout"
    # ---- columns, the exchange fused into the kernel: every rank stores its slab into every rank's buffer
    ctx.set_plan(0, variant=P.VARIANT_AUTO)
    gbuf = ctx.shard_alloc_gathered(world, M, n_loc)
    for it in range(3):
        gbuf.fill_(float("nan"))
        torch.cuda.synchronize()
        ctx.amm_column_sharded(0, x, gbuf, n_tokens=M, search_mode=P.SHARD_SEARCH_SPLIT, flags=P.FLAG_PEER_STORE)
        got = gbuf.permute(1, 0, 2).reshape(M, N).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (rank, it, "column-sharded, peer stores")
        dist.barrier()   # nobody refills its buffer while a peer may still be checking... its own copy only, but keep the ranks in step
    ctx.set_plan(0, variant=P.VARIANT_GATHER)   # no fused form: falls back to kernel + all-gather
    gbuf.fill_(float("nan"))
    torch.cuda.synchronize()
    ctx.amm_column_sharded(0, x, gbuf, n_tokens=M, flags=P.FLAG_PEER_STORE)
    assert np.array_equal(gbuf.permute(1, 0, 2).reshape(M, N).cpu().numpy().view(np.uint32), want.view(np.uint32)), "fallback"
    ctx.shard_free_gathered(gbuf)
    ctx.unload_weights(0)
    # a long codebook axis, so that tiles are split across CTAs and the summing pass does the peer stores
    c2 = synth.make_case(M=256 * world, K=2048, N=256 * world, v=2, CT=16, seed=4)
    want2 = oracle.amm(c2.x, c2.centroid, c2.lut, c2.bias, c2.scale, 0.0)[0]
    lo2, hi2 = shard.column_range(c2.N, rank, world)
    ctx.load_weights(2, c2.centroid, np.ascontiguousarray(c2.lut[:, :, lo2:hi2]), np.ascontiguousarray(c2.bias[lo2:hi2]), c2.scale)
    ctx.set_plan(2, variant=P.VARIANT_UMMA, umma_n_tile=128, umma_split=4)
    g2 = ctx.shard_alloc_gathered(world, c2.M, hi2 - lo2)
    g2.fill_(float("nan"))
    torch.cuda.synchronize()
    ctx.amm_column_sharded(2, torch.from_numpy(c2.x).cuda(), g2, n_tokens=c2.M, flags=P.FLAG_PEER_STORE)
    got2 = g2.permute(1, 0, 2).reshape(c2.M, c2.N).cpu().numpy()
    assert np.array_equal(got2.view(np.uint32), want2.view(np.uint32)), (rank, "peer stores, split tiles")
    ctx.shard_free_gathered(g2)
    ctx.unload_weights(2)
    # ---- tokens: weights replicated
    ctx.load_weights(1, c.centroid, c.lut, c.bias, c.scale)
    m_lo, m_hi = shard.token_range(M, rank, world)
    mine = torch.empty(m_hi - m_lo, N, device="cuda")
    ctx.amm_token_sharded(1, x[m_lo:m_hi].contiguous(), mine, M, gather=False)
    assert np.array_equal(mine.cpu().numpy().view(np.uint32), want[m_lo:m_hi].view(np.uint32)), (rank, "token-sharded")
    # a token count the ranks do not divide: near-equal blocks, the first ranks one row more
    M_odd = M - 1
    o_lo, o_hi = shard.token_range(M_odd, rank, world)
    odd = torch.empty(o_hi - o_lo, N, device="cuda")
    ctx.amm_token_sharded(1, x[o_lo:o_hi].contiguous(), odd, M_odd, gather=False)
    assert np.array_equal(odd.cpu().numpy().view(np.uint32), want[o_lo:o_hi].view(np.uint32)), (rank, "token-sharded, uneven")
    try:
        ctx.amm_token_sharded(1, x[o_lo:o_hi].contiguous(), odd, M_odd, gather=True)
        raise AssertionError("gathering uneven blocks must be refused")
    except P.LutAmmError:
        pass
    full = torch.full((M, N), float("nan"), device="cuda")
    ctx.amm_token_sharded(1, x[m_lo:m_hi].contiguous(), full, M, gather=True)
    assert np.array_equal(full.cpu().numpy().view(np.uint32), want.view(np.uint32)), (rank, "token-sharded + gather")
    gfull = ctx.shard_alloc_gathered(1, M, N)          # [1][M][N]: the full output, storable by every rank
    gfull.fill_(float("nan"))
    torch.cuda.synchronize()
    ctx.amm_token_sharded(1, x[m_lo:m_hi].contiguous(), gfull, M, gather=True, flags=P.FLAG_PEER_STORE)
    assert np.array_equal(gfull[0].cpu().numpy().view(np.uint32), want.view(np.uint32)), (rank, "token-sharded, peer stores")
    ctx.shard_free_gathered(gfull)
    # ---- which sharding is fastest here: every candidate timed, the same report on every rank
    ctx.load_weights(0, c.centroid, np.ascontiguousarray(c.lut[:, :, lo:hi]), np.ascontiguousarray(c.bias[lo:hi]), c.scale)
    rep = ctx.tune_sharding(1, 0, M, reps=2)
    assert rep["world"] == world and set(rep["ms"]) == set(P.SHARDING_MODES), rep
    assert all(t is not None and t > 0 for t in rep["ms"].values()), rep          # default plans: every candidate exists
    assert rep["best"] != "tokens_local" and rep["ms"][rep["best"]] == min(t for n, t in rep["ms"].items() if n != "tokens_local"), rep
    box = [None] * world
    dist.all_gather_object(box, rep)
    assert all(b == box[0] for b in box), box
    ctx.set_plan(0, variant=P.VARIANT_GATHER)                                       # no fused kernel for this plan
    rep = ctx.tune_sharding(-1, 0, M, reps=1)
    assert rep["ms"]["columns_fused"] is None and rep["ms"]["tokens_gathered"] is None and rep["ms"]["columns"] > 0, rep
    assert rep["best"] in ("columns", "columns_split"), rep
    ctx.shard_finalize()
    ctx.close()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: sharded results bit-identical to the oracle")


if __name__ == "__main__":
    main()
