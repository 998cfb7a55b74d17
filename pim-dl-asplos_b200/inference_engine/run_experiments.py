"""Sensitivity sweeps of the reference's artifact evaluation (asplos24-ae/sensitivity-analysis/
run_experiments.py:6-16 flags, :28-246 the four explorations) on the GPU path: one encoder layer per
point through run_layer.py's code, results as CSV (matplotlib is not a dependency here; the
reference plots speed-up over its CPU baseline, the CSV carries the same ratio).

    python run_experiments.py                                   # all four explorations
    python run_experiments.py --single_point --experiment_type centroid --model_type bert-large \\
                              --exploration_value 64
    python run_experiments.py --plot_only                        # re-emit the summary from saved CSVs

Points (asplos24-ae/sensitivity-analysis/configs/): seq 512 x batch 64 unless swept;
  sub-vector : v in {2,4,8,16,32}, 16 centroids             (bert-base, bert-large, vit-huge)
  centroid   : CT in {128,64,32,16,8}, v = 4                 (same three models)
  batch-size : batch in {8,16,32,64,128}, v = 4, CT = 16     (same three models)
  hidden-dim : token_dim in {1024,2048,2560,4096,5120}, 256 codebooks for token_dim, 1024 for 4x
The configs are generated here instead of being stored: on the GPU nothing in them but the shapes
matters (the reference's files differ only in hand-tuned UPMEM mapping keys).
"""
import argparse
import csv
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

MODELS = {  # network_params of configs/<model>/...: head_num, head_dim, token_dim, ffn_hidden_dim, layer_num
    "bert-base": (12, 64, 768, 3072, 12),
    "bert-large": (16, 64, 1024, 4096, 24),
    "vit-huge": (16, 80, 1280, 5120, 32),
}
HIDDEN = {1024: (16, 64, 24), 2048: (32, 64, 24), 2560: (32, 80, 32), 4096: (32, 128, 32), 5120: (40, 128, 40)}
SWEEPS = {"sub-vector": [2, 4, 8, 16, 32], "centroid": [128, 64, 32, 16, 8], "batch-size": [8, 16, 32, 64, 128],
          "hidden-dim": [1024, 2048, 2560, 4096, 5120]}
# seconds per layer of the reference's 40-thread CPU baseline, the denominators of its speed-up plots
# (run_experiments.py:29-33, 135-139, 188-194); measured on the reference authors' Xeon, not here
REFERENCE_CPU_S = {
    "layer": {"bert-base": 4.31126, "bert-large": 6.20743, "vit-huge": 7.59894},
    "batch-size": {"bert-base": {8: 0.325862, 16: 0.897627, 32: 1.73693, 64: 4.31126, 128: 6.98285},
                   "bert-large": {8: 0.537471, 16: 1.04923, 32: 2.32561, 64: 6.20743, 128: 11.2442},
                   "vit-huge": {8: 0.750662, 16: 1.54711, 32: 3.04215, 64: 7.59894, 128: 12.3811}},
}


def parse_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument('--plot_only', action='store_true', default=False)
    p.add_argument('--single_point', action='store_true', default=False)
    p.add_argument('--experiment_type', type=str, default='sub-vector', choices=list(SWEEPS))
    p.add_argument('--model_type', type=str, default='bert-base', choices=list(MODELS))
    p.add_argument('--exploration_value', type=int, default=0)
    p.add_argument('--out_dir', type=str, default=os.path.join(os.getcwd(), "sensitivity_results"))
    p.add_argument('--seq_len', type=int, default=512)
    p.add_argument('--batch_size', type=int, default=64)
    p.add_argument('--dry_run', action='store_true', help='write the generated configs, run nothing')
    return p.parse_args(argv)


def make_config(experiment: str, model: str, value: int, seq_len: int = 512, batch_size: int = 64) -> dict:
    """The transformer YAML (schema of configs/transformer_output_example.yaml) of one sweep point."""
    v, ct = 4, 16
    if experiment == "hidden-dim":
        heads, head_dim, layers = HIDDEN[value]
        dim, ffn = value, 4 * value
        cb = {"qkv": 256, "o": 256, "ffn1": 256, "ffn2": 1024}
    else:
        heads, head_dim, dim, ffn, layers = MODELS[model]
        if experiment == "sub-vector":
            v = value
        elif experiment == "centroid":
            ct = value
        elif experiment == "batch-size":
            batch_size = value
        cb = {"qkv": dim // v, "o": dim // v, "ffn1": dim // v, "ffn2": ffn // v}
    ker = {}
    for name in ("qkv", "o", "ffn1", "ffn2"):
        ker[f"{name}_scale"], ker[f"{name}_bias"] = 0.1, 0.2
        ker[f"{name}_num_codebook"], ker[f"{name}_num_centroid"] = cb[name], ct
    return {"network_params": dict(seq_len=seq_len, batch_size=batch_size, head_num=heads, head_dim=head_dim,
                                   token_dim=dim, ffn_hidden_dim=ffn, layer_num=layers),
            "system_params": dict(num_threads=40, gpu_device=0), "kernel_params": ker}


def reference_cpu_seconds(experiment, model, value):
    if experiment == "batch-size":
        return REFERENCE_CPU_S["batch-size"][model][value]
    if experiment in ("sub-vector", "centroid"):
        return REFERENCE_CPU_S["layer"][model]
    return None


def points(args):
    if args.single_point:
        return [(args.experiment_type, args.model_type if args.experiment_type != "hidden-dim" else "-",
                 args.exploration_value)]
    out = []
    for exp, values in SWEEPS.items():
        for model in (MODELS if exp != "hidden-dim" else ["-"]):
            out += [(exp, model, val) for val in values]
    return out


FIELDS = ["experiment", "model", "value", "seq_len", "batch_size", "tokens", "avg_inference_s", "tokens_per_s",
          "reference_cpu_s", "speedup_over_reference_cpu"]


def run_point(exp, model, value, args, cfg_dir):
    import yaml
    cfg = make_config(exp, model if model != "-" else "bert-base", value, args.seq_len, args.batch_size)
    path = os.path.join(cfg_dir, f"{exp}_{model}_{value}.yaml")
    with open(path, "w") as f:
        yaml.safe_dump(cfg, f, sort_keys=False)
    net = cfg["network_params"]
    row = dict(experiment=exp, model=model, value=value, seq_len=net["seq_len"], batch_size=net["batch_size"],
               tokens=net["seq_len"] * net["batch_size"])
    if args.dry_run:
        return row
    import run_layer
    r = run_layer.run(argparse.Namespace(transformer_config_file=path, need_compile=False, need_measure_energy=False,
                                         need_breakdown=False, breakdown_type=0, tune=False, model_weight_file=None,
                                         layers=None), whole_model=False)
    ref = reference_cpu_seconds(exp, model, value)
    full = (args.seq_len, args.batch_size) == (512, 64)   # the published baselines are for the full-size points
    row.update(avg_inference_s=r["avg_s"], tokens_per_s=r["tokens_per_s"], reference_cpu_s=ref if full else None,
               speedup_over_reference_cpu=(ref / r["avg_s"]) if (ref and full) else None)
    return row


def main(argv=None):
    args = parse_args(argv)
    os.makedirs(args.out_dir, exist_ok=True)
    csv_path = os.path.join(args.out_dir, "sensitivity.csv")
    if args.plot_only:
        with open(csv_path) as f:
            rows = list(csv.DictReader(f))
    else:
        rows = []
        cfg_dir = os.path.join(args.out_dir, "configs")
        os.makedirs(cfg_dir, exist_ok=True)
        pts = points(args)
        for i, (exp, model, value) in enumerate(pts):
            rows.append(run_point(exp, model, value, args, cfg_dir))
            print(f"{exp} exploration, {i + 1} of {len(pts)} jobs finished", flush=True)
        with open(csv_path, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=FIELDS)
            w.writeheader()
            w.writerows(rows)
    for r in rows:
        print(",".join(str(r.get(k, "")) for k in FIELDS))
    print("results written to", csv_path)
    return rows


if __name__ == "__main__":
    main()
