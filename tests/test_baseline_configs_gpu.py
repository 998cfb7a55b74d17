"""GPU parity at the sizes the benchmark runs: every linear of the five benchmark workloads,
on the plan the library picks by itself (LUTAMM_VARIANT_AUTO, what bench.py times) and on the
CUDA-core gather plan, through lutamm_amm_debug.

Bars (the reference's own check is amm_cpu + check_dpu_result, inference-engine/test/test_amm.cpp:126-213):
closest-centroid indices and int32 accumulators bit-exact, fp32 outputs bit-identical (stated tolerance
1e-5 relative).  Where the CPU oracle would take minutes for all rows, the indices are still compared for
ALL rows and the gather side is covered by (1) a strided row subsample against the oracle, (2) a checksum
over every row that does not depend on the size - sum_n acc[m][n] must equal the sum over codebooks of
the selected table rows' sums, computed in numpy int64 - and (3) the two GPU variants, which share no
code below the C ABI, agreeing on the full output.
"""
import numpy as np
import pytest

import oracle
import pim_dl_asplos_b200 as P
from pim_dl_asplos_b200 import synth

pytestmark = pytest.mark.gpu

RTOL = 1e-5


def _row_checksum(lut, idx):
    """sum_n acc[m][n] from the table's row sums: int64 [M]."""
    CB = lut.shape[0]
    rowsum = lut.sum(axis=2, dtype=np.int64)                     # [CB][CT]
    return rowsum[np.arange(CB)[None, :], idx.astype(np.int64)].sum(axis=1)


def _check_linear(ctx, M, K, N, v, CT, seed, stream, layer_id, sample_rows=None, full_oracle=False, must_include=()):
    import torch
    cen, lut, bias = synth.make_weights(K, N, v, CT, seed=seed, stream=stream)
    x = synth.make_input(M, K, seed=seed, stream=stream)
    CB = K // v
    ctx.load_weights(layer_id, cen, lut, bias, 0.01, 0.0)
    want_idx = oracle.index_calculation(x, cen).astype(np.uint8)  # all rows
    if full_oracle:
        rows = np.arange(M)
    else:
        rows = np.unique(np.concatenate([np.arange(0, M, max(1, M // sample_rows)), np.asarray(must_include, dtype=np.int64)]))
    want_out, _, want_acc = oracle.amm(x[rows], cen, lut, bias, 0.01, 0.0)
    checksum = _row_checksum(lut, want_idx)
    xd = torch.from_numpy(x).cuda()
    outs = {}
    for name, plan in (("auto", dict(variant=P.VARIANT_AUTO)), ("gather", dict(variant=P.VARIANT_GATHER, gather_cfg=2))):
        ctx.set_plan(layer_id, **plan)
        g_out, g_idx, g_acc = ctx.amm_debug(layer_id, x)
        assert np.array_equal(g_idx, want_idx), f"{name}: indices differ from the oracle"
        assert np.array_equal(g_acc[rows], want_acc), f"{name}: int32 accumulators differ on the compared rows"
        assert np.array_equal(g_acc.astype(np.int64).sum(axis=1), checksum), f"{name}: a row's accumulator checksum is off"
        np.testing.assert_allclose(g_out[rows], want_out, rtol=RTOL, atol=0, err_msg=name)
        assert np.array_equal(g_out[rows].view(np.uint32), want_out.view(np.uint32)), f"{name}: fp32 outputs not bit-identical"
        # the production call on device buffers (the call the benchmark times) gives the same bytes
        yd = torch.empty(M, N, device="cuda", dtype=torch.float32)
        ctx.amm_host(layer_id, xd, yd)
        outs[name] = yd
        assert np.array_equal(yd.cpu().numpy().view(np.uint32), g_out.view(np.uint32)), f"{name}: amm != amm_debug"
    assert torch.equal(outs["auto"].view(torch.int32), outs["gather"].view(torch.int32)), "GPU variants disagree"
    ctx.unload_weights(layer_id)


@pytest.mark.parametrize("li", range(4))
def test_c2_bert_base_layer_every_row(ctx, li):
    """Workload c2: M = 1024, QKV 768->2304, O 768->768, FFN1 768->3072, FFN2 3072->768 (the default plan splits
    FFN2's codebook axis three ways), v = 2, 16 centroids.  Every row against the oracle."""
    w = synth.WORKLOADS["c2"]
    _, K, N = w["linears"][li]
    _check_linear(ctx, w["M"], K, N, w["v"], w["CT"], seed=0, stream=li, layer_id=40 + li, full_oracle=True)


@pytest.mark.parametrize("li", range(4))
def test_c3_bert_large_layer(ctx, li):
    """Workload c3: M = 8192, v = 4 (256 / 1024 codebooks), 1024->3072 / 1024 / 4096 and 4096->1024: the register-path
    search kernel <4,16> at scale and 192-wide tensor-memory tiles with several tiles per CTA."""
    w = synth.WORKLOADS["c3"]
    _, K, N = w["linears"][li]
    _check_linear(ctx, w["M"], K, N, w["v"], w["CT"], seed=0, stream=li, layer_id=44 + li, sample_rows=256)


@pytest.mark.parametrize("li", range(4))
def test_c4_vit_layer_with_the_ragged_last_tile(ctx, li):
    """Workload c4: M = 12608 = 98.5 row tiles of 128.  The compared rows include all of the half-filled
    last tile, rows 12544...12607."""
    w = synth.WORKLOADS["c4"]
    _, K, N = w["linears"][li]
    _check_linear(ctx, w["M"], K, N, w["v"], w["CT"], seed=0, stream=li, layer_id=48 + li, sample_rows=256,
                  must_include=range(12544, 12608))


@pytest.mark.parametrize("v,CT", [(v, ct) for v in (2, 4, 8) for ct in (8, 16, 32)])
def test_c5_sweep_point_on_a_row_slab(ctx, v, CT):
    """Workload c5's nine (sub-vector length, centroid count) points, K = 4096, N = 16384, on an 8192-row slab
    (tokens are independent, so a slab exercises the same kernels, tiles and one-hot builders - two codebooks
    per 16-byte chunk at 8 centroids, two chunks per codebook at 32 - as all 65536 rows)."""
    _check_linear(ctx, 8192, 4096, 16384, v, CT, seed=0, stream=0, layer_id=60, sample_rows=64)


def test_out_of_range_indices_contribute_nothing(ctx):
    """lutamm_pim_lut takes caller-supplied indices: one that is >= num_centroid selects no table row in either
    kernel variant (the tcgen05 one-hot row is all zero, the gather kernel masks the loaded bytes)."""
    M, K, N, v, CT = 200, 128, 256, 2, 16
    CB = K // v
    c = synth.make_case(M=M, K=K, N=N, v=v, CT=CT, seed=5)
    rng = np.random.default_rng(5)
    idx = rng.integers(0, CT, (M, CB), dtype=np.uint8)
    bad = rng.random((M, CB)) < 0.1
    idx_bad = np.where(bad, rng.integers(CT, 256, (M, CB)).astype(np.uint8), idx)
    lut_pad = np.concatenate([c.lut, np.zeros((CB, 1, N), np.int8)], axis=1)       # row CT = "nothing"
    acc = oracle.lut_gather(np.where(bad, CT, idx).astype(np.uint16), lut_pad)
    want = oracle.dequant(acc, c.bias, CB, c.scale, 0.0)
    ctx.load_weights(12, c.centroid, c.lut, c.bias, c.scale)
    for plan in (dict(variant=P.VARIANT_GATHER), dict(variant=P.VARIANT_UMMA)):
        ctx.set_plan(12, **plan)
        y = np.zeros((M, N), dtype=np.float32)
        ctx.pim_lut(12, idx_bad, y)
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), plan
    ctx.unload_weights(12)
