"""Checkpoint converter: a calibrated LUT-NN model (safetensors) -> the `.npz` the inference
engine loads.  Same command line and same output keys as the reference's
model-calibration/pim_weight_converter.py (flags :8-18, key handling :39-97, output :101-118);
the table construction (bmm + symmetric int8 quantisation, :21-36 and :83-91) runs on the GPU
through `lutamm_build_lut`.

    python weight_converter.py --weight_input_file model.safetensors --features 768 \\
        --ncentroids 16 --vec_len 2 --weight_output_file model.npz

For every encoder-layer linear `<L>.<op>` with a `.centroids.weight` beside its `.weight`, the
dense weight is replaced by `<L>.<op>.lut.tensor` (int8 [CB*CT][N]), `.lut.scale` and `.lut.bias`;
every other tensor of the layer passes through; embeddings and heads are dropped, as there.
There is no CPU path: without the CUDA library and a GPU the conversion fails.
"""
from __future__ import annotations

import argparse
import re

import numpy as np


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--weight_input_file", type=str, required=True)
    p.add_argument("--features", type=int, default=768)
    p.add_argument("--ncentroids", type=int, default=16)
    p.add_argument("--vec_len", type=int, default=2)
    p.add_argument("--nsharecodebook", type=int, default=1)
    p.add_argument("--weight_output_file", type=str, required=True)
    p.add_argument("--device", type=int, default=0, help="CUDA device that builds the tables")
    return p.parse_args(argv)


def read_checkpoint(path: str) -> dict:
    """All tensors of a safetensors file (or of an .npz with the same keys) as numpy arrays."""
    if path.endswith(".npz"):
        with np.load(path) as z:
            return {k: z[k] for k in z.files}
    from safetensors import safe_open
    out = {}
    with safe_open(path, framework="np") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k)
    return out


def group_layers(tensors: dict) -> dict:
    """{layer id: {short key: tensor}} with the key cut at the layer index, e.g.
    `bert.encoder.layer.3.output.dense.bias` -> `3.output.dense.bias` (pim_weight_converter.py:43-53)."""
    layers: dict[str, dict] = {}
    for k, t in tensors.items():
        parts = k.split(".")
        if "embeddings" in parts or "layer" not in parts:
            continue
        layer_id = parts[3]
        short = re.sub(".*" + str(layer_id), str(layer_id), k, count=1)
        layers.setdefault(layer_id, {})[short] = t
    return layers


def linear_shape(op_name: str, features: int):
    """in/out features from the operator's name (pim_weight_converter.py:72-79)."""
    fin = features if ("attention" in op_name or "intermediate" in op_name) else features * 4
    fout = features if ("attention" in op_name or "output" in op_name) else features * 4
    return fin, fout


def convert(tensors: dict, features: int, ncentroids: int, vec_len: int, nsharecodebook: int = 1, ctx=None,
            device: int = 0) -> dict:
    """The converted tensor dictionary; `ctx` is an open LutAmmContext (one is made if absent)."""
    from . import LutAmmContext
    own = ctx is None
    if own:
        ctx = LutAmmContext(device)
    try:
        out = {}
        for layer_id, lt in group_layers(tensors).items():
            lt = dict(lt)
            ops = [k[:-len(".centroids.weight")] for k in lt if k.endswith(".centroids.weight")]
            for op in ops:
                if op + ".weight" not in lt:
                    raise KeyError(f"{op}: centroids without a dense weight")
                fin, fout = linear_shape(op, features)
                CB = fin // vec_len // nsharecodebook
                weight = np.ascontiguousarray(lt.pop(op + ".weight"), dtype=np.float32)
                centroid = np.ascontiguousarray(lt[op + ".centroids.weight"], dtype=np.float32)
                if weight.size != CB * vec_len * fout or centroid.size != CB * ncentroids * vec_len:
                    raise ValueError(f"{op}: tensor sizes do not match features={features}, vec_len={vec_len}, "
                                     f"ncentroids={ncentroids}, nsharecodebook={nsharecodebook}")
                lut, scale, lut_bias = ctx.build_lut(centroid.reshape(CB, ncentroids, vec_len),
                                                     weight.reshape(CB * vec_len, fout))
                lt[op + ".lut.tensor"] = lut.reshape(CB * ncentroids, fout)
                lt[op + ".lut.scale"] = np.float32(scale)
                lt[op + ".lut.bias"] = np.float32(lut_bias)
            out.update(lt)
        return out
    finally:
        if own:
            ctx.close()


def store(path: str, tensors: dict) -> None:
    np.savez(path, **tensors)
    with np.load(path if path.endswith(".npz") else path + ".npz") as back:   # the reference re-reads its dump (:108-114)
        for name, t in tensors.items():
            if name not in back.files:
                print("warning, %s not exist in dumped file" % name)
            elif not np.array_equal(t, back[name]):
                print("warning, %s not equal in dumped file" % name)
    print("dump finished")


def main(argv=None):
    args = parse_args(argv)
    tensors = read_checkpoint(args.weight_input_file)
    store(args.weight_output_file, convert(tensors, args.features, args.ncentroids, args.vec_len, args.nsharecodebook,
                                           device=args.device))


if __name__ == "__main__":
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pim_dl_asplos_b200  # noqa: F401
    from pim_dl_asplos_b200 import weight_converter as _wc
    _wc.main()
