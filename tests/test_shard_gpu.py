"""The sharded forms of the operator on real GPUs, through the C ABI (lutamm_amm_column_sharded,
lutamm_amm_token_sharded), against the CPU oracle's unsharded result, bit for bit.  Needs two or more
GPUs for the exchange itself; the world-size-1 path of the same calls runs on one."""
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle
import pim_dl_asplos_b200 as P
from pim_dl_asplos_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_world_size_one_is_the_plain_operator(ctx):
    import torch
    c = synth.make_case(M=300, K=256, N=512, v=2, CT=16, seed=4)
    want = oracle.amm(c.x, c.centroid, c.lut, c.bias, c.scale, 0.0)[0]
    ctx.load_weights(20, c.centroid, c.lut, c.bias, c.scale)
    x = torch.from_numpy(c.x).cuda()
    y = torch.empty(1, 300, 512, device="cuda")
    for mode in (P.SHARD_SEARCH_REPLICATED, P.SHARD_SEARCH_SPLIT):
        ctx.amm_column_sharded(20, x, y, search_mode=mode)
        assert np.array_equal(y[0].cpu().numpy().view(np.uint32), want.view(np.uint32))
    y2 = torch.empty(300, 512, device="cuda")
    ctx.amm_token_sharded(20, x, y2, 300, gather=True)
    assert np.array_equal(y2.cpu().numpy().view(np.uint32), want.view(np.uint32))
    with pytest.raises(P.LutAmmError):
        ctx.amm_column_sharded(20, c.x, y)          # host buffers are refused
    rep = ctx.tune_sharding(20, 20, 512)            # one GPU: nothing to fuse, every other candidate is timed
    assert rep["world"] == 1 and rep["ms"]["tokens_fused"] is None and rep["ms"]["columns_fused"] is None
    assert all(rep["ms"][n] > 0 for n in ("tokens_local", "tokens_gathered", "columns", "columns_split")), rep
    assert rep["best"] in ("tokens_gathered", "columns", "columns_split")
    with pytest.raises(P.LutAmmError):
        ctx.tune_sharding(-1, -1, 512)
    with pytest.raises(P.LutAmmError):
        ctx.tune_sharding(20, 99, 512)
    ctx.unload_weights(20)


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_results_equal_the_unsharded_oracle(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + world), os.path.join(ROOT, "tests", "shard_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("bit-identical to the oracle") == world
