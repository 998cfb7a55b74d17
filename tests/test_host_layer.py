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
    transformer_config.save_with_plans(raw, {"ffn1": {"variant": 2, "umma_n_tile": 192, "umma_operand": 2, "umma_epilogue": 1}}, str(out))
    cfg, _ = transformer_config.load(str(out))
    assert cfg["plans"] == {"ffn1": {"variant": 2, "umma_n_tile": 192, "umma_operand": 2, "umma_epilogue": 1}}


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


LAYER = textwrap.dedent("""\
    network_params:
      seq_len: 64
      batch_size: 8
      head_num: 4
      head_dim: 64
      token_dim: 256
      ffn_hidden_dim: 1024
      layer_num: 3

    system_params:
      dpu_num: 64
      nr_tasklets: 16
      qkv_lut_pim_binary: "./build/bin/dpu_bin_qkv"
      o_lut_pim_binary: "./build/bin/dpu_bin_o"
      ffn1_lut_pim_binary: "./build/bin/dpu_bin_ffn1"
      ffn2_lut_pim_binary: "./build/bin/dpu_bin_ffn2"
      num_threads: 40

    kernel_params:
    """) + "".join(textwrap.indent(textwrap.dedent(f"""\
      {p}_scale: 0.1
      {p}_bias: 0.2
      {p}_num_codebook: {cb}
      {p}_num_centroid: 16
      {p}_input_parallelism: 8
      {p}_lut_parallelism: 8
      {p}_loop_order: 0
      {p}_lut_load_type: 2
      {p}_n_mtile_size: 32
      {p}_feature_mtile_size: 32
      {p}_cb_mtile_size: 32
      {p}_feature_load_tile_size: 8
      {p}_cb_load_tile_size: 32
    """), "  ") for p, cb in (("qkv", 64), ("o", 64), ("ffn1", 64), ("ffn2", 256)))


def test_cpp_transformer_parser_reads_the_reference_schema(tmp_path):
    """parse_transformer_configs (src/host/parser.cpp:89-413) in C++, through the layer driver: the reference's
    full schema incl. the UPMEM mapping keys, derived values, and FFN2 as ffn_hidden_dim -> token_dim."""
    cfg = tmp_path / "layer.yaml"
    cfg.write_text(LAYER)
    r = run("test_transformer_layer", str(cfg))
    assert "layer num 3" in r.stdout and "thread num 40" in r.stdout
    assert "n 512, input feature len 256, output feature len 768" in r.stdout        # QKV: 3 x token_dim
    assert "n 512, input feature len 1024, output feature len 256" in r.stdout       # FFN2
    assert "num codebook 256, num centroid 16, sub vec len 4" in r.stdout
    assert "scale 0.1, bias 0.2" in r.stdout
    assert "head num 4, head dim 64, token dim 256" in r.stdout
    if not torch.cuda.is_available():
        assert r.returncode == 1 and "cannot create a GPU context" in r.stderr


@pytest.mark.parametrize("edit,msg", [
    (("ffn2_num_codebook: 256", "ffn2_num_codebook: 100"), "ffn2: input feature length is not a multiple of num_codebook"),
    (("head_dim: 64", "head_dim: 48"), "head_dim * head_num != token_dim"),
    (("  o_input_parallelism: 8", "  o_input_parallelism: 16"), "o: input_parallelism * lut_parallelism != dpu_num"),
    (("  ffn1_cb_load_tile_size: 32", "  ffn1_cb_load_tile_size: 5"), "ffn1: cb_mtile_size % cb_load_tile_size"),
    (("  o_loop_order: 0", "  o_loop_order: 0\n  o_gpu_umma_epilogue: copy"), "kernel_params.o_gpu_umma_epilogue: not an unsigned integer"),
    (("  qkv_num_centroid: 16\n", ""), "missing kernel_params.qkv_num_centroid"),
    (("  seq_len: 64\n", ""), "missing network_params.seq_len"),
])
def test_cpp_transformer_parser_rejects_bad_configs(tmp_path, edit, msg):
    cfg = tmp_path / "bad.yaml"
    assert edit[0] in LAYER
    cfg.write_text(LAYER.replace(*edit))
    r = run("test_transformer_layer", str(cfg))
    assert r.returncode == 2, r.stdout + r.stderr
    assert msg in r.stderr


def test_cpp_transformer_parser_accepts_the_shipped_configs():
    for name, want in (("bert_base_layer.yaml", "n 1024, input feature len 3072, output feature len 768"),
                       ("bert_large_layer.yaml", "n 8192, input feature len 4096, output feature len 1024"),
                       ("vit_base_model.yaml", "layer num 12")):
        r = run("test_transformer_layer", os.path.join(CFG, name))
        assert want in r.stdout, r.stdout + r.stderr


def test_search_space_sweep_points():
    """The plan-space sweep that stands for asplos24-ae/search-space-illustration: every exploration lists its
    points without a GPU, the global table is the union without duplicates."""
    sys.path.insert(0, os.path.join(PKG, "inference_engine"))
    import search_space as ss
    pts = ss.main(["--dry_run"])
    assert set(pts) == set(ss.EXPERIMENTS)
    assert "2-192" in pts["operand-tile"] and "1-256" in pts["operand-tile"] and len(pts["gather"]) == 5
    assert len(pts["global"]) == len(set(pts["global"])) >= 25
    assert ss.SHAPE == dict(n=32768, K=1024, N=4096, CB=256, CT=16)
