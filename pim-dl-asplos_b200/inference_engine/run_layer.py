"""Encoder-layer launcher with the reference's command line (inference-engine/run_layer.py:7-16):

    python run_layer.py --transformer_config_file configs/bert_base_layer.yaml
                        [--need_compile] [--need_breakdown --breakdown_type {0,1,2}] [--tune]

Runs 5 warm-up and 10 timed rounds of one layer (test_transformer_layer.cpp:35-36) on random
weights and prints "inference time", the line the reference's experiment scripts look for,
plus tokens/s.  --need_breakdown prints the per-linear times in the reference's wording
("qkv projection time ..."): breakdown types 0/1/2 select AMM stage / AMM-vs-rest / per-linear
there (run_layer.py:132-152); here one timed pass reports all of them.
--need_measure_energy is accepted; RAPL through `sudo rdmsr` has no GPU counterpart and is
reported as unsupported.
"""
import argparse
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
sys.path.insert(0, os.path.dirname(PKG))
sys.path.insert(0, HERE)

WARMUP_ROUND, RECORD_ROUND = 5, 10


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument('--transformer_config_file', type=str, required=True)
    p.add_argument('--need_compile', action='store_true', default=True)
    p.add_argument('--need_measure_energy', action='store_true', default=False)
    p.add_argument('--need_breakdown', action='store_true', default=False)
    p.add_argument('--breakdown_type', type=int, default=0)
    p.add_argument('--tune', action='store_true', default=False)
    p.add_argument('--model_weight_file', type=str, default=None)
    p.add_argument('--layers', type=int, default=None, help='override layer_num (run_layer: 1)')
    p.add_argument('--separate_qkv', action='store_true', default=False,
                   help='run Q, K and V as three operators (the reference model driver\'s SEPARATE build, run_model.py:130); '
                        'a checkpoint that holds query/key/value instead of a fused qkv operator selects this by itself')
    p.add_argument('--separate_gelu', action='store_true', default=False,
                   help='run GELU as its own pass after FFN1, as the reference does, instead of in the FFN1 epilogue')
    return p.parse_args()


def run(args, whole_model: bool):
    import numpy as np
    import torch
    import transformer_config
    import pim_dl_asplos_b200 as P
    from pim_dl_asplos_b200 import build, layer as L

    if args.need_compile:
        build.build_all()
    if args.need_measure_energy:
        print("energy measurement: unsupported on this backend (the reference reads RAPL MSRs of the host CPU)")
    cfg, raw = transformer_config.load(args.transformer_config_file)
    n_layers = (args.layers or cfg["layer_num"]) if whole_model else 1
    S, B, H, D, F = cfg["seq_len"], cfg["batch_size"], cfg["head_num"], cfg["token_dim"], cfg["ffn_hidden_dim"]
    n = S * B
    torch.cuda.set_device(cfg["gpu_device"])
    ctx = P.LutAmmContext(cfg["gpu_device"])
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)

    npz = None
    if args.model_weight_file and os.path.exists(args.model_weight_file):
        npz = np.load(args.model_weight_file)
        print("loading weights from", args.model_weight_file)
    elif args.model_weight_file:
        print("weight file not found, using random weights (as test_transformer.cpp:484-489 does)")
    weights = []
    if npz is not None:
        n_layers = min(n_layers, L.checkpoint_layer_count(npz)) or n_layers
    for li in range(n_layers):
        if npz is not None:
            weights.append(L.load_layer_weights_npz(npz, li, D, F, cfg["num_codebook"], cfg["num_centroid"],
                                                    separate_qkv=True if args.separate_qkv else None))
        else:
            w = L.random_layer_weights(D, F, cfg["num_codebook"], cfg["num_centroid"], seed=0, layer=li,
                                       separate_qkv=args.separate_qkv)
            for name in (L.SEPARATE_LINEARS if args.separate_qkv else L.LINEARS):
                cen, lut, bias, _, _ = w[name]
                key = name if name in cfg["scale"] else "o"
                w[name] = (cen, lut, bias, cfg["scale"][key], cfg["lut_bias"][key])
            weights.append(w)
    print("attention projections:", "separate Q / K / V operators" if "qkv" not in weights[0] else "one fused QKV operator")
    model = L.LutTransformer(ctx, weights, S, B, H, plans=cfg["plans"], fused_gelu=not getattr(args, "separate_gelu", False))
    if args.tune:
        plans = model.layers[0].tune()
        for lay in model.layers[1:]:
            for name in lay.linears:
                ctx.set_plan(lay.ids[name], **plans[name])
        out = os.path.splitext(args.transformer_config_file)[0] + ".tuned.yaml"
        transformer_config.save_with_plans(raw, plans, out)
        print("tuned plans written to", out)

    x = torch.from_numpy(L.synth.make_input(n, D, seed=0)).cuda()
    total = 0.0
    with torch.cuda.stream(stream):
        for rnd in range(WARMUP_ROUND + RECORD_ROUND):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            y = model.forward(x)
            e1.record(stream)
            stream.synchronize()
            ctx.sync()
            t = e0.elapsed_time(e1) * 1e-3
            print(f"---------- ROUND {rnd} ----------")
            print(f"inference time {t:.6f}")
            if rnd >= WARMUP_ROUND:
                total += t
    avg = total / RECORD_ROUND
    print(f"warm up rounds {WARMUP_ROUND}, record rounds {RECORD_ROUND}")
    print(f"AVG inference time {avg:.6f}")
    print(f"tokens per second {n / avg:.1f}" + (f", images per second {B / avg:.1f}" if whole_model else ""))
    print(f"output checksum {float(y.double().sum()):.6e}")

    if args.need_breakdown:
        ctx.enable_timing(True)
        names = {"qkv": "qkv projection", "q": "q projection", "k": "k projection", "v": "v projection",
                 "o": "o projection", "ffn1": "ffn1", "ffn2": "ffn2"}
        lay = model.layers[0]
        inputs = {"qkv": x, "q": x, "k": x, "v": x, "o": x, "ffn1": x, "ffn2": torch.zeros(n, F, device="cuda")}
        amm_total = 0.0
        for name in lay.linears:
            ctx.amm_host(lay.ids[name], inputs[name], lay.buf[name], n_tokens=n)
            t = ctx.timings()
            amm_total += t["total_ms"]
            print(f"{names[name]} time {t['total_ms'] * 1e-3:.6f} (index calculation {t['index_calc_ms'] * 1e-3:.6f}, "
                  f"lut kernel {t['lut_kernel_ms'] * 1e-3:.6f})")
        print(f"amm time {amm_total * 1e-3 * n_layers:.6f}, non-amm time {max(avg - amm_total * 1e-3 * n_layers, 0):.6f}")
        ctx.enable_timing(False)
    ctx.close()
    return {"avg_s": avg, "tokens": n, "tokens_per_s": n / avg}


if __name__ == '__main__':
    run(parse_args(), whole_model=False)
