"""CPU checks of the oracle: against the committed golden vectors (generated from the
reference's own index_calc_host.cpp), against an independent numpy statement, and - when
oracle/_ref is present - directly against the reference object on more shapes."""
import numpy as np
import pytest

import oracle
from conftest import golden_names, load_golden
from pim_dl_asplos_b200 import synth


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_golden(name):
    g = load_golden(name)
    out, idx, acc = oracle.amm(g["x"], g["centroid"], g["lut"], g["bias"], float(g["scale"]), float(g["lut_bias"]))
    assert np.array_equal(idx, g["idx"]), "closest-centroid indices differ from the reference's"
    assert np.array_equal(acc, g["acc"])
    # bit-exact: same operations, same order, fp32 each
    assert np.array_equal(out.view(np.uint32), g["out"].view(np.uint32))


@pytest.mark.parametrize("name", golden_names())
def test_numpy_statement_matches_golden(name):
    g = load_golden(name)
    assert np.array_equal(oracle.numpy_index_calculation(g["x"], g["centroid"]), g["idx"])


def test_golden_adversarial_cases_exercise_the_hysteresis():
    """A plain argmin must disagree with the reference on the adversarial fixtures,
    otherwise they would not pin the sequential epsilon scan."""
    total = 0
    for name in ("adversarial_v2_ct16", "adversarial_v4_ct8"):
        g = load_golden(name)
        x, c = g["x"], g["centroid"]
        M, K = x.shape
        CB, CT, v = c.shape
        d = ((x.reshape(M, CB, 1, v).astype(np.float64) - c[None].astype(np.float64)) ** 2).sum(-1)
        total += int((d.argmin(-1) != g["idx"]).sum())
    assert total > 50


def test_golden_tiled_layout():
    g = load_golden("tiled_v2_ct16")
    flat = oracle.index_calculation_tiled(g["x"], g["centroid"], int(g["n_stile"]), int(g["cb_mtile"]))
    assert np.array_equal(flat, g["idx_tiled"])
    M, CB = g["idx"].shape
    assert np.array_equal(oracle.untile_index(flat, M, CB, int(g["n_stile"]), int(g["cb_mtile"])), g["idx"])


@pytest.mark.skipif(not oracle.have_reference(), reason="oracle/_ref not built (reference tree absent)")
@pytest.mark.parametrize("M,K,v,CT,style", [
    (512, 768, 2, 16, False), (256, 1024, 4, 16, False), (128, 512, 8, 32, False), (64, 256, 2, 8, False),
    (100, 96, 2, 16, True), (31, 160, 16, 128, False), (16, 64, 32, 64, False), (7, 30, 3, 7, False),
])
def test_restatement_equals_reference_object(M, K, v, CT, style):
    c = synth.make_case(M=M, K=K, N=16, v=v, CT=CT, seed=1234 + M, reference_style=style)
    ref = oracle.ref_index_calculation(c.x, c.centroid).reshape(M, K // v)
    mine = oracle.index_calculation(c.x, c.centroid)
    assert np.array_equal(ref, mine)


@pytest.mark.skipif(not oracle.have_reference(), reason="oracle/_ref not built (reference tree absent)")
def test_restatement_equals_reference_object_tiled():
    c = synth.make_case(M=128, K=128, N=16, v=2, CT=16, seed=5)
    ref = oracle.ref_index_calculation(c.x, c.centroid, n_stile=32, cb_mtile=16)
    mine = oracle.index_calculation_tiled(c.x, c.centroid, 32, 16)
    assert np.array_equal(ref, mine)
    assert np.array_equal(oracle.untile_index(ref, 128, 64, 32, 16), oracle.index_calculation(c.x, c.centroid))


def test_empty_inputs():
    c = synth.make_case(M=0, K=32, N=16, v=2, CT=8, seed=1)
    out, idx, acc = oracle.amm(c.x, c.centroid, c.lut, c.bias, c.scale)
    assert out.shape == (0, 16) and idx.shape == (0, 16) and acc.shape == (0, 16)


def test_gather_extremes_and_linearity():
    """All -128 entries over the largest codebook count of any benchmark shape stay exact
    in int32; gathering is additive over a split of the codebook axis."""
    CB, CT, N, M = 2048, 4, 16, 3
    lut = np.full((CB, CT, N), -128, dtype=np.int8)
    idx = np.zeros((M, CB), dtype=np.uint16)
    assert (oracle.lut_gather(idx, lut) == -128 * CB).all()
    rng = np.random.default_rng(0)
    lut = rng.integers(-128, 128, (CB, CT, N), dtype=np.int8)
    idx = rng.integers(0, CT, (M, CB)).astype(np.uint16)
    whole = oracle.lut_gather(idx, lut)
    parts = oracle.lut_gather(idx[:, :1000], lut[:1000]) + oracle.lut_gather(idx[:, 1000:], lut[1000:])
    assert np.array_equal(whole, parts)


def test_dequant_follows_production_expression():
    """(float)acc*scale + lut_bias*CB + bias, left to right (pim_lut_host.cpp:201); the
    reference's own checker adds lut_bias once instead (test_amm.cpp:181) - they agree only
    for lut_bias == 0, which is what converted weights always have."""
    rng = np.random.default_rng(3)
    acc = rng.integers(-50000, 50000, (5, 32)).astype(np.int32)
    bias = rng.standard_normal(32).astype(np.float32)
    scale, lb, CB = np.float32(0.1), np.float32(0.2), 256
    want = ((acc.astype(np.float32) * scale + lb * np.float32(CB)).astype(np.float32) + bias).astype(np.float32)
    got = oracle.dequant(acc, bias, CB, float(scale), float(lb))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(oracle.dequant(acc, bias, CB, float(scale), 0.0),
                          oracle.dequant_checker_variant(acc, bias, float(scale), 0.0))
    assert not np.allclose(got, oracle.dequant_checker_variant(acc, bias, float(scale), float(lb)))


def test_tiled_output_offsets_are_a_permutation():
    M, N, n_stile, f_stile, f_mtile = 32, 64, 8, 16, 4
    lut_par = N // f_stile
    offs = {oracle.tiled_output_offset(i, j, n_stile, f_stile, f_mtile, lut_par) for i in range(M) for j in range(N)}
    assert offs == set(range(M * N))
    # first DPU, first micro-tile: rows of f_mtile consecutive features
    assert oracle.tiled_output_offset(0, 1, n_stile, f_stile, f_mtile, lut_par) == 1
    assert oracle.tiled_output_offset(1, 0, n_stile, f_stile, f_mtile, lut_par) == f_mtile


def test_reorder_lut_roundtrip():
    rng = np.random.default_rng(1)
    CB, CT, N, tile = 6, 4, 32, 8
    lut = rng.integers(-128, 128, (CB, CT, N), dtype=np.int8)
    t = oracle.reorder_lut(lut, tile).reshape(N // tile, CB, CT, tile)
    assert np.array_equal(t.transpose(1, 2, 0, 3).reshape(CB, CT, N), lut)


def test_gelu_checker_properties():
    """The activation checker: known points of the tanh-form GELU, its limits, and the fp16-table
    form's defining property (every output is an fp16 value; inputs that round to the same fp16 value
    give the same output)."""
    x = np.array([0.0, 1.0, -1.0, 3.0, -3.0, 10.0, -10.0], np.float32)
    g = oracle.gelu_tanh(x)
    np.testing.assert_allclose(g[:5], [0.0, 0.8411920, -0.1588080, 2.9963627, -0.0036373], rtol=0, atol=2e-7)
    assert g[5] == 10.0 and abs(g[6]) < 1e-20
    rng = np.random.default_rng(0)
    y = rng.normal(0, 2, 4096).astype(np.float32)
    h = oracle.gelu_tanh(y, through_f16=True)
    assert np.array_equal(h, h.astype(np.float16).astype(np.float32))
    assert np.array_equal(h, oracle.gelu_tanh(y.astype(np.float16).astype(np.float32), through_f16=True))
    np.testing.assert_allclose(h, oracle.gelu_tanh(y), rtol=2e-3, atol=1e-3)
