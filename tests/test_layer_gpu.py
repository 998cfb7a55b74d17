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
