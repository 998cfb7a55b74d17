"""Generates converter_checkpoint.npz + converter_reference_output.npz in this directory.  Run from the
repository root in a container that has the reference tree mounted:

    python tests/golden/make_converter_golden.py

A tiny synthetic LUT-NN checkpoint (one encoder layer, hidden size 32, sub-vector 2, 16 centroids, key
names as the reference's converter expects them) is written as safetensors to a temporary file and
run through the REFERENCE's own model-calibration/pim_weight_converter.py (read_weight + store_weight,
imported from the reference tree, unmodified; the only change is that its safetensors reader is asked
for CPU tensors because this container has no GPU).  The checkpoint tensors and the reference's output
are committed so the converter of this repository can be checked without the reference tree.
"""
import argparse
import importlib.util
import os
import tempfile

import numpy as np

OUT = os.path.dirname(os.path.abspath(__file__))
# the reference tree: $LUTAMM_REFERENCE_DIR, else a checkout named `reference` beside this repository
REF = os.environ.get("LUTAMM_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(OUT))), "reference")

FEATURES, VEC_LEN, NCENT = 32, 2, 16
LINEARS = {  # name -> (in_features, out_features), pim_weight_converter.py:72-79
    "attention.self.query": (FEATURES, FEATURES), "attention.self.key": (FEATURES, FEATURES),
    "attention.self.value": (FEATURES, FEATURES), "attention.output.dense": (FEATURES, FEATURES),
    "intermediate.dense": (FEATURES, 4 * FEATURES), "output.dense": (4 * FEATURES, FEATURES),
}


def synthetic_checkpoint(seed=7):
    rng = np.random.default_rng(seed)
    t = {}
    p = "bert.encoder.layer.0."
    for name, (fin, fout) in LINEARS.items():
        t[p + name + ".weight"] = rng.normal(0, 0.05, (fin, fout)).astype(np.float32)
        t[p + name + ".bias"] = rng.normal(0, 0.02, (fout,)).astype(np.float32)
        t[p + name + ".centroids.weight"] = rng.normal(0, 1, (fin // VEC_LEN, NCENT, VEC_LEN)).astype(np.float32)
    for ln in ("attention.output.LayerNorm", "output.LayerNorm"):
        t[p + ln + ".weight"] = rng.uniform(0.5, 1.5, (FEATURES,)).astype(np.float32)
        t[p + ln + ".bias"] = rng.normal(0, 0.1, (FEATURES,)).astype(np.float32)
    t["bert.embeddings.word_embeddings.weight"] = rng.normal(0, 1, (8, FEATURES)).astype(np.float32)
    return t


def main():
    import safetensors
    from safetensors.numpy import save_file
    spec = importlib.util.spec_from_file_location("ref_converter", os.path.join(REF, "model-calibration/pim_weight_converter.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    ref.safe_open = lambda f, framework, device: safetensors.safe_open(f, framework=framework, device="cpu")

    ckpt = synthetic_checkpoint()
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "model.safetensors")
        dst = os.path.join(tmp, "converted.npz")
        save_file(ckpt, src)
        args = argparse.Namespace(weight_input_file=src, features=FEATURES, ncentroids=NCENT, vec_len=VEC_LEN,
                                  nsharecodebook=1, weight_output_file=dst)
        ref.store_weight(args, ref.read_weight(args))
        converted = dict(np.load(dst))
    np.savez_compressed(os.path.join(OUT, "converter_checkpoint.npz"), **ckpt)
    np.savez_compressed(os.path.join(OUT, "converter_reference_output.npz"), **converted)
    print("checkpoint keys:", len(ckpt), " converted keys:", len(converted))
    for k in sorted(converted)[:8]:
        print(" ", k, converted[k].shape, converted[k].dtype)


if __name__ == "__main__":
    main()
