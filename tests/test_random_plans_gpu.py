"""Seeded random shapes x random plans of the tcgen05 kernel against the oracle: tile width, operand
placement, split, builder groups, slabs per turn and ring depth drawn independently, so that the
launcher's own adjustments (ring slot ownership, one CTA per SM, odd items) are exercised in
combinations no hand-written case lists.  Indices, int32 accumulators and fp32 outputs bit-exact."""
import numpy as np
import pytest

import oracle
import pim_dl_asplos_b200 as P
from pim_dl_asplos_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_shapes_and_plans(ctx, seed):
    rng = np.random.default_rng(1000 + seed)
    shapes = 0
    while shapes < 6:
        CT = int(rng.choice([8, 16, 16, 32, 64, 128]))
        v = int(rng.choice([2, 4, 8]))
        CB = 16 * int(rng.integers(1, 49))
        N = 16 * int(rng.integers(1, 200))
        M = int(rng.choice([rng.integers(1, 300), rng.integers(300, 2600), 128 * rng.integers(1, 24)]))
        if M * N * CB > 6e8:
            continue
        shapes += 1
        c = synth.make_case(M=M, K=CB * v, N=N, v=v, CT=CT, seed=int(rng.integers(1 << 30)))
        out, idx, acc = oracle.amm(c.x, c.centroid, c.lut, c.bias, c.scale, 0.0)
        ctx.load_weights(5, c.centroid, c.lut, c.bias, c.scale)
        for _ in range(8):
            op = int(rng.choice([0, 1, 2, 2]))
            tiles = {0: [0], 1: [0, 64, 128, 256], 2: [0, 64, 128, 160, 192]}[op]
            plan = dict(variant=P.VARIANT_UMMA, umma_operand=op, umma_n_tile=int(rng.choice(tiles)),
                        umma_split=int(rng.choice([0, 0, 1, 2, 3, 4, 5, 7, 12])), umma_groups=int(rng.integers(0, 5)),
                        umma_sps=int(rng.choice([0, 1, 2, 4])), umma_epilogue=int(rng.choice([0, 1, 2, 2])),
                        umma_stages=int(rng.choice([0, 0, 2, 3, 4, 5, 7, 9, 12, 13, 16])))
            ctx.set_plan(5, **plan)
            for _rep in range(2):
                g_out, g_idx, g_acc = ctx.amm_debug(5, c.x)
                where = f"M={M} CB={CB} v={v} CT={CT} N={N} {plan}"
                assert np.array_equal(g_idx, idx.astype(np.uint8)), where
                assert np.array_equal(g_acc, acc), where
                assert np.array_equal(g_out.view(np.uint32), out.view(np.uint32)), where
            y = np.zeros_like(out)                 # the production call: no int32 copy, so the plan's epilogue form runs
            ctx.amm_host(5, c.x, y)
            assert np.array_equal(y.view(np.uint32), out.view(np.uint32)), "amm_host: " + where
        ctx.unload_weights(5)
