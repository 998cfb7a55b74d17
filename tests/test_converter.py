"""Weight converter (model-calibration/pim_weight_converter.py of the reference): the CPU restatement
against the reference's own output on a committed synthetic checkpoint, the host-side key handling,
and (GPU) the CUDA table construction against both."""
import numpy as np
import pytest

import oracle
import pim_dl_asplos_b200 as P
from conftest import GOLDEN_DIR
from pim_dl_asplos_b200 import weight_converter as wc

FEATURES, VEC_LEN, NCENT = 32, 2, 16   # the shape tests/golden/make_converter_golden.py used


def fixtures():
    import os
    ck = dict(np.load(os.path.join(GOLDEN_DIR, "converter_checkpoint.npz")))
    ref = dict(np.load(os.path.join(GOLDEN_DIR, "converter_reference_output.npz")))
    return ck, ref


def test_restatement_matches_the_reference_converter_output():
    ck, ref = fixtures()
    ops = [k[:-len(".lut.tensor")] for k in ref if k.endswith(".lut.tensor")]
    assert len(ops) == 6
    for op in ops:
        w = ck["bert.encoder.layer." + op + ".weight"]
        c = ck["bert.encoder.layer." + op + ".centroids.weight"]
        lut, scale, lut_bias = oracle.build_lut(c, w)
        want = ref[op + ".lut.tensor"]
        assert want.dtype == np.int8 and want.shape == (c.shape[0] * NCENT, w.shape[1])
        # the reference's bmm order is its BLAS's; one int8 step at rounding boundaries is the stated bar
        d = np.abs(lut.reshape(want.shape).astype(np.int32) - want.astype(np.int32))
        assert d.max() <= 1 and (d > 0).mean() < 1e-3
        np.testing.assert_allclose(scale, ref[op + ".lut.scale"], rtol=1e-6)
        assert float(lut_bias) == 0.0 and float(ref[op + ".lut.bias"]) == 0.0
        assert np.abs(lut).max() == 127


def test_key_grouping_and_shapes():
    ck, ref = fixtures()
    layers = wc.group_layers(ck)
    assert list(layers) == ["0"]
    assert "0.output.dense.centroids.weight" in layers["0"] and not any("embeddings" in k for k in layers["0"])
    assert wc.linear_shape("0.attention.self.query", 768) == (768, 768)
    assert wc.linear_shape("0.intermediate.dense", 768) == (768, 3072)
    assert wc.linear_shape("0.output.dense", 768) == (3072, 768)
    # pass-through keys of the reference's output are exactly the non-weight keys of the layer
    passthrough = {k for k in ref if ".lut." not in k}
    assert passthrough == {k for k in layers["0"] if not (k.endswith(".weight") and k[:-7] + ".centroids.weight" in layers["0"])}


def test_zero_table_has_zero_scale():
    lut, scale, _ = oracle.build_lut(np.zeros((4, 8, 2), np.float32), np.ones((8, 16), np.float32))
    assert scale == 0 and not lut.any()


@pytest.mark.gpu
def test_gpu_converter_matches_reference_and_restatement(ctx, tmp_path):
    ck, ref = fixtures()
    got = wc.convert(ck, FEATURES, NCENT, VEC_LEN, ctx=ctx)
    assert set(got) == set(ref)
    for k, want in ref.items():
        g = np.asarray(got[k])
        if k.endswith(".lut.tensor"):
            op = k[:-len(".lut.tensor")]
            mine, scale, _ = oracle.build_lut(ck["bert.encoder.layer." + op + ".centroids.weight"],
                                              ck["bert.encoder.layer." + op + ".weight"])
            assert np.array_equal(g, mine.reshape(g.shape)), f"{k}: CUDA table differs from the stated order"
            assert np.float32(got[op + ".lut.scale"]) == scale
            d = np.abs(g.astype(np.int32) - want.astype(np.int32))
            assert g.dtype == np.int8 and g.shape == want.shape and d.max() <= 1 and (d > 0).mean() < 1e-3
        elif k.endswith(".lut.scale"):
            np.testing.assert_allclose(g, want, rtol=1e-6)
        else:
            assert np.array_equal(g, want), k
    # round trip through the file format and the layer loader
    path = str(tmp_path / "converted.npz")
    wc.store(path, got)
    back = np.load(path)
    assert set(back.files) == set(ref)


@pytest.mark.gpu
@pytest.mark.parametrize("CB,CT,v,N", [(384, 16, 2, 3072), (96, 32, 8, 768), (64, 8, 4, 20), (5, 5, 3, 36), (8, 256, 1, 64), (12, 16, 20, 64), (4, 16, 32, 128)])
def test_gpu_build_lut_shapes(ctx, CB, CT, v, N):
    """Bit-exact against the stated order on BERT-base FFN1 and odd shapes; device-resident operands too."""
    import torch
    rng = np.random.default_rng(CB + N)
    cen = rng.normal(0, 1, (CB, CT, v)).astype(np.float32)
    w = rng.normal(0, 0.05, (CB * v, N)).astype(np.float32)
    want, scale, lut_bias = oracle.build_lut(cen, w)
    lut, s, b = ctx.build_lut(cen, w)
    assert np.array_equal(lut, want) and np.float32(s) == scale and b == 0.0
    d_lut = torch.empty((CB, CT, N), dtype=torch.int8, device="cuda")
    _, s2, _ = ctx.build_lut(torch.from_numpy(cen).cuda(), torch.from_numpy(w).cuda(), d_lut)
    assert np.array_equal(d_lut.cpu().numpy(), want) and np.float32(s2) == scale
    # the table it builds drives the operator: dequantised AMM output approximates x @ w
    if N % 16 == 0 and CT <= 256:
        x = cen[np.arange(CB)[None, :], rng.integers(0, CT, (32, CB))].reshape(32, CB * v)  # rows made of centroids
        bias = np.zeros(N, np.float32)
        ctx.load_weights(9, cen, lut, bias, s, b)
        y = np.zeros((32, N), np.float32)
        ctx.amm_host(9, np.ascontiguousarray(x), y)
        ctx.unload_weights(9)
        exact = x.astype(np.float64) @ w.astype(np.float64)
        assert np.abs(y - exact).max() <= 0.5 * s * CB + 1e-4   # at most half a quantisation step per codebook


@pytest.mark.gpu
def test_gpu_build_lut_rejects_bad_shapes(ctx):
    with pytest.raises(P.LutAmmError) as e:
        ctx.build_lut(np.zeros((4, 8, 2), np.float32), np.zeros((8, 18), np.float32))
    assert e.value.code == P.EINVAL
    with pytest.raises(P.LutAmmError):   # one codebook's centroids must fit 48 KB of shared memory
        ctx.build_lut(np.zeros((1, 256, 64), np.float32), np.zeros((64, 16), np.float32))


def test_layer_loader_reads_what_the_converters_write():
    """The layer loader against the reference converter's own output file (no GPU needed): a converted
    checkpoint holds the three projections query / key / value - there is no fused qkv operator in it - so the
    layer is loaded with separate Q / K / V operators (the reference's SEPARATE build reads the same keys,
    test/test_transformer.cpp:295-368), with the attention-output operator's codebook settings
    (src/host/parser.cpp:235-322)."""
    from pim_dl_asplos_b200 import layer as L
    _, ref = fixtures()
    D, F = FEATURES, 4 * FEATURES
    cb = {"qkv": 16, "o": 16, "ffn1": 16, "ffn2": 64}
    ct = {k: NCENT for k in cb}
    w = L.load_layer_weights_npz(ref, 0, D, F, cb, ct)
    assert set(w) == {"q", "k", "v", "o", "ffn1", "ffn2", "ln1", "ln2"}
    for name, (K, N, CB) in {"q": (D, D, 16), "k": (D, D, 16), "v": (D, D, 16), "o": (D, D, 16), "ffn1": (D, F, 16), "ffn2": (F, D, 64)}.items():
        cen, lut, bias, scale, lut_bias = w[name]
        assert cen.shape == (CB, NCENT, K // CB) and lut.shape == (CB, NCENT, N) and lut.dtype == np.int8 and bias.shape == (N,)
        assert scale > 0 and lut_bias == 0.0
    assert np.array_equal(w["q"][1].reshape(-1, D), ref["0.attention.self.query.lut.tensor"])
    assert L.checkpoint_layer_count(ref) == 1
    with pytest.raises(KeyError):
        L.load_layer_weights_npz(ref, 0, D, F, cb, ct, separate_qkv=False)      # no fused operator in this file
    with pytest.raises(ValueError):
        L.load_layer_weights_npz(ref, 0, D, F, dict(cb, o=8), ct)               # wrong codebook count
    # a file with a fused operator loads as one
    fused = dict(ref)
    for suffix in ("centroids.weight", "lut.scale", "lut.bias"):
        fused["0.attention.self.qkv." + suffix] = ref["0.attention.self.query." + suffix]
    fused["0.attention.self.qkv.lut.tensor"] = np.concatenate([ref[f"0.attention.self.{n}.lut.tensor"] for n in ("query", "key", "value")], axis=1)
    fused["0.attention.self.qkv.bias"] = np.concatenate([ref[f"0.attention.self.{n}.bias"] for n in ("query", "key", "value")])
    w2 = L.load_layer_weights_npz(fused, 0, D, F, cb, ct)
    assert "qkv" in w2 and w2["qkv"][1].shape == (16, NCENT, 3 * D)
