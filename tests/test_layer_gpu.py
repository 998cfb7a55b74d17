"""GPU checks of the callers of the hot path: the encoder layer (four AMMs + dense
attention / LayerNorm / GELU in PyTorch) and the launchers."""
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle
import pim_dl_asplos_b200 as P
from pim_dl_asplos_b200 import layer as L

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "pim-dl-asplos_b200")


@pytest.mark.parametrize("fused_gelu", [False, True])
def test_encoder_layer_follows_the_reference_dataflow(ctx, fused_gelu):
    """Every AMM inside the layer is bit-exact against the oracle on the very input the GPU
    layer fed it (so index flips cannot hide or appear through float noise upstream), and
    the layer output matches a numpy statement of transformer_layer.cpp:263-625 to 1e-4 -
    the tolerance covers the dense fp32 parts, which the reference runs in ggml and whose
    rounding is not pinned."""
    import torch
    S, B, H, D, F = 16, 4, 4, 64, 128
    cb = {"qkv": 32, "o": 32, "ffn1": 32, "ffn2": 64}
    ct = {k: 16 for k in cb}
    w = L.random_layer_weights(D, F, cb, ct, seed=5)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    lay = L.LutTransformerLayer(ctx, w, S, B, H, first_layer_id=40, fused_gelu=fused_gelu)
    x = L.synth.make_input(S * B, D, seed=5)
    seen = {}
    orig = lay._amm

    def spy(name, t):
        out = orig(name, t)
        ctx.sync()
        seen[name] = (t.detach().cpu().numpy().copy(), out.detach().cpu().numpy().copy())
        return out

    lay._amm = spy
    with torch.cuda.stream(stream):
        y = lay.forward(torch.from_numpy(x).cuda())
    stream.synchronize()
    for name in L.LINEARS:
        xin, got = seen[name]
        cen, lut, bias, scale, lb = w[name]
        want, _, _ = oracle.amm(xin, cen, lut, bias, scale, lb)
        if name == "ffn1" and fused_gelu:
            # GELU applied in the operator's epilogue: a float function of a bit-exact value
            # (hardware exp2 / reciprocal approximations against float64 numpy), rel 1e-5 / abs 1e-9
            np.testing.assert_allclose(got, oracle.gelu_tanh(want), rtol=1e-5, atol=1e-9)
            continue
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name

    def amm(name, t):
        cen, lut, bias, scale, lb = w[name]
        return oracle.amm(t, cen, lut, bias, scale, lb)[0]

    ref = L.reference_layer_numpy(x, w, S, B, H, amm)
    np.testing.assert_allclose(y.cpu().numpy(), ref, rtol=1e-4, atol=1e-4)
    ctx.set_stream(None)
    for lid in lay.ids.values():
        ctx.unload_weights(lid)


def test_run_amm_launcher():
    r = subprocess.run([sys.executable, os.path.join(PKG, "inference_engine", "run_amm.py"), "--amm_config_file",
                        os.path.join(PKG, "inference_engine", "configs", "bert_base_ffn1_amm.yaml"), "--need_breakdown"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "PIM AVG AMM time" in r.stdout and "index calculation time" in r.stdout


def test_run_layer_launcher():
    r = subprocess.run([sys.executable, os.path.join(PKG, "inference_engine", "run_layer.py"), "--transformer_config_file",
                        os.path.join(PKG, "inference_engine", "configs", "bert_base_layer.yaml"), "--need_breakdown"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "AVG inference time" in r.stdout and "qkv projection time" in r.stdout


def test_tuner_cli_writes_a_config_the_driver_accepts(tmp_path):
    src = tmp_path / "in.yaml"
    src.write_text(open(os.path.join(PKG, "inference_engine", "configs", "bert_base_ffn1_amm.yaml")).read())
    out = tmp_path / "out.yaml"
    r = subprocess.run([os.path.join(PKG, "bin", "tuner"), "0", str(src), str(out)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    text = out.read_text()
    assert "gpu_variant" in text and "n_stile_size" in text
    r = subprocess.run([os.path.join(PKG, "bin", "test_amm"), str(out)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "PIM AVG AMM time" in r.stdout


def test_converted_checkpoint_runs_end_to_end(ctx, tmp_path):
    """Checkpoint -> weight_converter.convert -> .npz -> layer loader -> encoder layer, the path
    run_model.py --model_weight_file takes.  The converter writes the three projections query / key / value
    (pim_weight_converter.py:56-96), so the layer runs them as three operators, as the reference's SEPARATE
    build does (transformer_layer.cpp:333-343; keys read at test_transformer.cpp:295-368).  Run on the file
    the REFERENCE converter wrote for the same checkpoint (tests/golden/converter_reference_output.npz), every
    AMM inside the layer is bit-exact against the oracle on the very input the GPU layer fed it; run on the
    file this repository's converter wrote, the tables are identical, the quantisation scales agree to 1e-6
    (the reference's bmm sums in its BLAS's order) and the layer output agrees to 1e-5."""
    import torch
    from conftest import GOLDEN_DIR
    from pim_dl_asplos_b200 import weight_converter as wc
    ck = dict(np.load(os.path.join(GOLDEN_DIR, "converter_checkpoint.npz")))
    ref = np.load(os.path.join(GOLDEN_DIR, "converter_reference_output.npz"))
    D, F, H, S, B = 32, 128, 4, 8, 4
    cb = {"qkv": 16, "o": 16, "ffn1": 16, "ffn2": 64}
    ct = {k: 16 for k in cb}
    path = str(tmp_path / "converted.npz")
    wc.store(path, wc.convert(ck, D, 16, 2, ctx=ctx))
    mine = L.load_layer_weights_npz(np.load(path), 0, D, F, cb, ct)
    theirs = L.load_layer_weights_npz(ref, 0, D, F, cb, ct)
    assert "qkv" not in mine and set(mine) == set(theirs) == {"q", "k", "v", "o", "ffn1", "ffn2", "ln1", "ln2"}
    with pytest.raises(KeyError):
        L.load_layer_weights_npz(ref, 0, D, F, cb, ct, separate_qkv=False)
    for name in L.SEPARATE_LINEARS:   # this checkpoint's tables come out identical to the reference converter's
        assert np.array_equal(mine[name][1], theirs[name][1]) and mine[name][3] == pytest.approx(theirs[name][3], rel=1e-6)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    model = L.LutTransformer(ctx, [theirs], S, B, H, fused_gelu=False)
    lay = model.layers[0]
    assert lay.separate_qkv
    x = L.synth.make_input(S * B, D, seed=9)
    seen, orig = {}, lay._amm

    def spy(name, t):
        out = orig(name, t)
        ctx.sync()
        seen[name] = (t.detach().cpu().numpy().copy(), out.detach().cpu().numpy().copy())
        return out

    lay._amm = spy
    with torch.cuda.stream(stream):
        y = model.forward(torch.from_numpy(x).cuda())
    stream.synchronize()
    for name in L.SEPARATE_LINEARS:
        xin, got = seen[name]
        cen, lut, bias, scale, lb = theirs[name]
        want = oracle.amm(xin, cen, lut, bias, scale, lb)[0]
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name

    def amm(name, t):
        cen, lut, bias, scale, lb = theirs[name]
        return oracle.amm(t, cen, lut, bias, scale, lb)[0]

    np.testing.assert_allclose(y.cpu().numpy(), L.reference_layer_numpy(x, theirs, S, B, H, amm), rtol=1e-4, atol=1e-4)
    for lid in lay.ids.values():
        ctx.unload_weights(lid)
    model2 = L.LutTransformer(ctx, [mine], S, B, H, fused_gelu=False)
    with torch.cuda.stream(stream):
        y2 = model2.forward(torch.from_numpy(x).cuda())
    stream.synchronize()
    np.testing.assert_allclose(y2.cpu().numpy(), y.cpu().numpy(), rtol=1e-5, atol=1e-6)
    ctx.set_stream(None)
    for lid in model2.layers[0].ids.values():
        ctx.unload_weights(lid)
    # the launcher on this repository's converted file
    cfg = tmp_path / "tiny.yaml"
    cfg.write_text("network_params:\n  seq_len: 8\n  batch_size: 4\n  head_num: 4\n  head_dim: 8\n  token_dim: 32\n  ffn_hidden_dim: 128\n"
                   "  layer_num: 1\nsystem_params:\n  num_threads: 1\nkernel_params:\n" +
                   "".join(f"  {n}_num_codebook: {cb[n]}\n  {n}_num_centroid: 16\n" for n in ("qkv", "o", "ffn1", "ffn2")))
    r = subprocess.run([sys.executable, os.path.join(PKG, "inference_engine", "run_model.py"), "--transformer_config_file", str(cfg),
                        "--model_weight_file", path], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "separate Q / K / V operators" in r.stdout and "AVG inference time" in r.stdout


def test_run_model_launcher_with_separate_projections():
    r = subprocess.run([sys.executable, os.path.join(PKG, "inference_engine", "run_model.py"), "--transformer_config_file",
                        os.path.join(PKG, "inference_engine", "configs", "bert_base_layer.yaml"), "--separate_qkv", "--need_breakdown"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "AVG inference time" in r.stdout and "q projection time" in r.stdout and "v projection time" in r.stdout


def test_tuner_mode_1_and_the_cpp_layer_driver(tmp_path):
    """`tuner 1` (the reference's tune_single_model, src/tuner/auto_tuner.cpp:745-790) tunes the four linears of a
    layer and writes a YAML both the C++ layer driver (parse_transformer_configs) and run_layer.py accept; the
    plans are also kept by shape beside it and a second run finds them there."""
    src = os.path.join(PKG, "inference_engine", "configs", "bert_base_layer.yaml")
    out = tmp_path / "tuned.yaml"
    r = subprocess.run([os.path.join(PKG, "bin", "tuner"), "1", src, str(out)], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout + r.stderr
    text = out.read_text()
    assert all(f"{p}_gpu_variant" in text for p in ("qkv", "o", "ffn1", "ffn2")) and "ffn2_cb_mtile_size" in text
    cache = (tmp_path / "tuned.yaml.plans").read_text()
    assert len([ln for ln in cache.splitlines() if ln and not ln.startswith("#")]) == 4
    r = subprocess.run([os.path.join(PKG, "bin", "test_transformer_layer"), str(out)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "rounds' average inference time" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
    r = subprocess.run([os.path.join(PKG, "bin", "test_transformer_layer"), str(out), "--separate"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "separate Q / K / V" in r.stdout
    r = subprocess.run([sys.executable, os.path.join(PKG, "inference_engine", "run_layer.py"), "--transformer_config_file", str(out)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "AVG inference time" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]


def test_search_space_sweep_single_point_and_experiment(tmp_path):
    eng = os.path.join(PKG, "inference_engine")
    r = subprocess.run([sys.executable, os.path.join(eng, "search_space.py"), "--single_point", "--experiment_type", "operand-tile",
                        "--exploration_value", "2-192", "--tokens", "4096"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "PIM AVG AMM time" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
    sys.path.insert(0, eng)
    import search_space as ss
    bench = ss.Bench(4096, 0)
    rows = ss.run_experiment(bench, "gather", str(tmp_path))
    bench.ctx.close()
    assert len(rows) == 5 and all(r["amm_time_s"] > 0 for r in rows) and (tmp_path / "gather.csv").exists()
