"""Reads the transformer YAML of the reference (configs/transformer_output_example.yaml,
parsed there by parse_transformer_configs(), src/host/parser.cpp:89-413)."""
import yaml

LINEARS = ("qkv", "o", "ffn1", "ffn2")
PLAN_KEYS = ("variant", "ccs_tokens", "gather_cfg", "umma_n_tile", "umma_split", "umma_stages", "umma_groups", "umma_operand", "umma_sps", "umma_epilogue")


def load(path):
    with open(path) as f:
        y = yaml.safe_load(f)
    net, ker = y["network_params"], y.get("kernel_params", {})
    sysp = y.get("system_params", {})
    cfg = dict(seq_len=int(net["seq_len"]), batch_size=int(net["batch_size"]), head_num=int(net["head_num"]),
               token_dim=int(net["token_dim"]), ffn_hidden_dim=int(net["ffn_hidden_dim"]), layer_num=int(net.get("layer_num", 1)),
               gpu_device=int(sysp.get("gpu_device", 0)))
    if "head_dim" in net and int(net["head_dim"]) * cfg["head_num"] != cfg["token_dim"]:
        raise ValueError("head_dim * head_num != token_dim")
    dims = {"qkv": cfg["token_dim"], "o": cfg["token_dim"], "ffn1": cfg["token_dim"], "ffn2": cfg["ffn_hidden_dim"]}
    cfg["num_codebook"], cfg["num_centroid"], cfg["scale"], cfg["lut_bias"], cfg["plans"] = {}, {}, {}, {}, {}
    for name in LINEARS:
        cb = int(ker[f"{name}_num_codebook"])
        if dims[name] % cb:
            raise ValueError(f"{name}: input feature length {dims[name]} is not a multiple of num_codebook {cb}")  # parser.cpp:395-410
        cfg["num_codebook"][name] = cb
        cfg["num_centroid"][name] = int(ker[f"{name}_num_centroid"])
        cfg["scale"][name] = float(ker.get(f"{name}_scale", 0.01))
        cfg["lut_bias"][name] = float(ker.get(f"{name}_bias", 0.0))
        plan = {k: int(ker[f"{name}_gpu_{k}"]) for k in PLAN_KEYS if f"{name}_gpu_{k}" in ker}
        if plan:
            cfg["plans"][name] = plan
    for name in ("q", "k", "v"):   # separate projections: shapes from the attention-output keys (parser.cpp:235-322), own plans if tuned
        plan = {k: int(ker[f"{name}_gpu_{k}"]) for k in PLAN_KEYS if f"{name}_gpu_{k}" in ker}
        if plan:
            cfg["plans"][name] = plan
    return cfg, y


def save_with_plans(y, plans, path):
    ker = y.setdefault("kernel_params", {})
    for name, plan in plans.items():
        for k, v in plan.items():
            ker[f"{name}_gpu_{k}"] = int(v)
    with open(path, "w") as f:
        yaml.safe_dump(y, f, sort_keys=False)
