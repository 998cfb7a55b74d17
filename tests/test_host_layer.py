"""CPU checks of the C++ host layer above the C ABI (YAML parser, test_amm driver, tuner
CLI) and of the Python launchers' configuration reader.  No GPU work: on a machine without
a device the drivers must stop with a clear message after parsing."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "pim-dl-asplos_b200")
BIN = os.path.join(PKG, "bin")
CFG = os.path.join(PKG, "inference_engine", "configs")

pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(BIN, "test_amm")),
                                reason="host layer not built (run __graft_entry__.build())")

FULL = textwrap.dedent("""\
    system_params:
      # for cpu
      num_threads: 40
      # for dpu
      dpu_num: 64
      nr_tasklets: 16

    amm_shape_params:
      num_codebook: 64
      num_centroid: 16
      n: 512
      input_feature_len: 256
      output_feature_len: 1024
      scale: 0.1   # trailing comment
      bias: 0.2

    kernel_params:
      loop_order: 1
      lut_load_type: 2
      n_stile_size: 64
      feature_stile_size: 128
      n_mtile_size: 32
      feature_mtile_size: 32
      cb_mtile_size: 32
      feature_load_tile_size: 8
      cb_load_tile_size: 16
    """)


def run(exe, *args):
    return subprocess.run([os.path.join(BIN, exe), *args], capture_output=True, text=True, timeout=120)


def test_driver_parses_the_reference_schema(tmp_path):
    cfg = tmp_path / "k.yaml"
    cfg.write_text(FULL)
    r = run("test_amm", str(cfg), "dpu_bin_ignored")
    assert "num codebook 64, num centroid 16" in r.stdout
    assert "n 512, input feature len 256, output feature len 1024" in r.stdout
    assert "sub vec len 4, input parallelism 8, lut parallelism 8" in r.stdout   # parser.cpp:26,41-42
    assert "scale 0.1, bias 0.2" in r.stdout
    if not torch.cuda.is_available():
        assert r.returncode == 1 and "cannot create a GPU context" in r.stderr


@pytest.mark.parametrize("edit,msg", [
    (("num_codebook: 64", "num_codebook: 60"), "not a multiple of num_codebook"),           # parser.cpp:57
    (("dpu_num: 64", "dpu_num: 100"), "input_parallelism * lut_parallelism != dpu_num"),     # parser.cpp:59
    (("n_mtile_size: 32", "n_mtile_size: 24"), "n_stile_size % n_mtile_size"),               # parser.cpp:62
    (("cb_load_tile_size: 16", "cb_load_tile_size: 5"), "cb_mtile_size % cb_load_tile_size"),  # parser.cpp:66
    (("  scale: 0.1   # trailing comment\n", ""), "missing amm_shape_params.scale"),
    (("n: 512", "n: many"), "not an unsigned integer"),
])
def test_driver_rejects_bad_configs(tmp_path, edit, msg):
    cfg = tmp_path / "bad.yaml"
    cfg.write_text(FULL.replace(*edit))
    r = run("test_amm", str(cfg))
    assert r.returncode == 2, r.stdout + r.stderr
    assert msg in r.stderr


def test_missing_file_and_usage():
    assert run("test_amm").returncode == 2
    r = run("test_amm", "/nonexistent.yaml")
    assert r.returncode == 2 and "cannot open" in r.stderr
    assert run("tuner", "1", "a", "b").returncode == 2


def test_shipped_amm_configs_parse():
    for name in ("bert_base_ffn1_amm.yaml", "large_amm.yaml"):
        r = run("test_amm", os.path.join(CFG, name))
        assert "sub vec len 2" in r.stdout, r.stderr


def test_transformer_configs_load():
    sys.path.insert(0, os.path.join(PKG, "inference_engine"))
    import transformer_config
    cfg, _ = transformer_config.load(os.path.join(CFG, "bert_base_layer.yaml"))
    assert cfg["seq_len"] * cfg["batch_size"] == 1024 and cfg["token_dim"] == 768
    assert cfg["num_codebook"] == {"qkv": 384, "o": 384, "ffn1": 384, "ffn2": 1536}
    cfg, _ = transformer_config.load(os.path.join(CFG, "bert_large_layer.yaml"))
    assert cfg["num_codebook"]["ffn2"] == 1024 and cfg["seq_len"] * cfg["batch_size"] == 8192
    cfg, raw = transformer_config.load(os.path.join(CFG, "vit_base_model.yaml"))
    assert cfg["layer_num"] == 12 and cfg["seq_len"] * cfg["batch_size"] == 12608


def test_tuned_plans_round_trip(tmp_path):
    sys.path.insert(0, os.path.join(PKG, "inference_engine"))
    import transformer_config
    _, raw = transformer_config.load(os.path.join(CFG, "bert_base_layer.yaml"))
    out = tmp_path / "t.yaml"
    transformer_config.save_with_plans(raw, {"ffn1": {"variant": 2, "umma_n_tile": 192, "umma_operand": 2}}, str(out))
    cfg, _ = transformer_config.load(str(out))
    assert cfg["plans"] == {"ffn1": {"variant": 2, "umma_n_tile": 192, "umma_operand": 2}}


def test_sensitivity_sweep_configs(tmp_path):
    """The artifact-evaluation sweep driver generates the reference's shapes
    (asplos24-ae/sensitivity-analysis/configs) and every config passes the transformer parser."""
    import os
    import sys
    eng = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "pim-dl-asplos_b200", "inference_engine")
    sys.path.insert(0, eng)
    import run_experiments as rx
    import transformer_config
    rows = rx.main(["--dry_run", "--out_dir", str(tmp_path)])
    assert len(rows) == 3 * 5 * 3 + 5
    c = rx.make_config("sub-vector", "bert-base", 8)
    assert c["kernel_params"]["qkv_num_codebook"] == 96 and c["kernel_params"]["ffn2_num_codebook"] == 384
    c = rx.make_config("centroid", "bert-base", 128)
    assert c["kernel_params"]["o_num_codebook"] == 192 and c["kernel_params"]["o_num_centroid"] == 128
    c = rx.make_config("hidden-dim", "-", 5120)
    assert c["network_params"]["head_num"] * c["network_params"]["head_dim"] == 5120
    assert c["kernel_params"]["ffn2_num_codebook"] == 1024 and c["network_params"]["ffn_hidden_dim"] == 20480
    c = rx.make_config("batch-size", "vit-huge", 8)
    assert c["network_params"]["batch_size"] == 8 and c["kernel_params"]["qkv_num_codebook"] == 320
    for f in os.listdir(tmp_path / "configs"):
        cfg, _ = transformer_config.load(str(tmp_path / "configs" / f))
        assert cfg["token_dim"] % cfg["num_codebook"]["qkv"] == 0
    assert rx.reference_cpu_seconds("batch-size", "bert-large", 32) == 2.32561
