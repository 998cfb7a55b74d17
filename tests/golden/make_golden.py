"""Generates the golden vectors in this directory.  Run from the repository root, in a
container that has the reference tree mounted:

    make -C oracle && python tests/golden/make_golden.py

For every case the closest-centroid indices come from the REFERENCE's own, unmodified
inference-engine/src/host/index_calc_host.cpp (compiled into oracle/_ref by
oracle/Makefile and called through oracle/ref_shim.cpp).  The int32 accumulators and fp32
outputs are then derived from those reference indices by exact integer addition and by
the dequantisation expression of inference-engine/src/host/pim_lut_host.cpp:201, evaluated
with numpy fp32 scalars (one rounding per operation) - independently of the C oracle, so
that the oracle is checked against these files rather than against itself.

The `refamm_*` files additionally hold `out_ref` / `out_ref_tiled`: the output of the reference's
WHOLE operator - amm_host.cpp, index_calc_host.cpp, pim_lut_host.cpp and the DPU kernel
src/dpu/pim_lut_kernel.c, all unmodified - run on host threads through the functional UPMEM
stand-in in oracle/upmem_shim (row-major, and in the DPU-tiled order the reference returns), with
the mapping parameters stored beside them.  The generator asserts that it is bit-identical to the
numpy derivation above.

Each .npz holds the inputs too, so the fixtures are self-contained on machines without
the reference tree.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
import pim_dl_asplos_b200  # noqa: E402,F401
from pim_dl_asplos_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def derive(idx, lut, bias, scale, lut_bias):
    M, CB = idx.shape
    _, CT, N = lut.shape
    acc = np.zeros((M, N), dtype=np.int64)
    for cb in range(CB):
        acc += lut[cb, idx[:, cb].astype(np.int64), :].astype(np.int64)
    acc = acc.astype(np.int32)
    a = acc.astype(np.float32) * np.float32(scale)
    b = np.float32(lut_bias) * np.float32(CB)
    out = ((a + b).astype(np.float32) + bias[None, :]).astype(np.float32)
    return acc, out


def adversarial(M, CB, CT, v, seed):
    """Ties and near-epsilon gaps: grid-valued data gives exact distance ties (lowest index
    must win); a second family puts pairs of centroids a hair apart so that distance gaps
    straddle the 1e-6 hysteresis threshold in both directions."""
    rng = np.random.default_rng(seed)
    cent = (rng.integers(-4, 5, (CB, CT, v)) * 0.25).astype(np.float32)
    x = (rng.integers(-8, 9, (M, CB * v)) * 0.125).astype(np.float32)
    # duplicate centroids -> exact ties between different indices
    for cb in range(0, CB, 3):
        cent[cb, CT - 1] = cent[cb, 0]
        cent[cb, CT // 2] = cent[cb, 1]
    # near-epsilon family on every 4th codebook: centroid c = base + c*delta in dim 0
    for cb in range(1, CB, 4):
        base = np.float32(0.01)
        delta = rng.uniform(2e-5, 1e-4)
        for c in range(CT):
            cent[cb, c, :] = 0
            cent[cb, c, 0] = np.float32(base + (CT - 1 - c) * delta)  # distances shrink slowly with c
        x[:, cb * v:(cb + 1) * v] = (rng.uniform(-1e-3, 1e-3, (M, v))).astype(np.float32)
    return x, cent


def emit(name, x, cent, lut, bias, scale, lut_bias, n_stile=None, cb_mtile=None):
    M, K = x.shape
    CB, CT, v = cent.shape
    flat = oracle.ref_index_calculation(x, cent, n_stile, cb_mtile, nthreads=4)
    if n_stile:
        idx = oracle.untile_index(flat, M, CB, n_stile, cb_mtile)
        extra = dict(idx_tiled=flat, n_stile=n_stile, cb_mtile=cb_mtile)
    else:
        idx = flat.reshape(M, CB)
        extra = {}
    acc, out = derive(idx, lut, bias, scale, lut_bias)
    np.savez_compressed(os.path.join(OUT, name + ".npz"), x=x, centroid=cent, lut=lut, bias=bias,
                        scale=np.float32(scale), lut_bias=np.float32(lut_bias), idx=idx, acc=acc, out=out, **extra)
    print(f"{name}: M={M} K={K} v={v} CT={CT} N={lut.shape[2]} idx-hist-head={np.bincount(idx.ravel(), minlength=CT)[:4]}")


def emit_refamm(name, case_name, seed, scale, lut_bias, reference_style=False):
    cfg = dict(oracle.REF_AMM_CASES[case_name])
    M, N, CB, CT, v = (cfg[k] for k in ("M", "N", "CB", "CT", "v"))
    c = synth.make_case(M=M, K=CB * v, N=N, v=v, CT=CT, seed=seed, scale=scale, lut_bias=lut_bias,
                        reference_style=reference_style)
    r = oracle.ref_amm_case(case_name, scale=scale, lut_bias=lut_bias, nthreads=4)
    tiled = r.run_tiled(c.x, c.centroid, r.dpu_lut(c.lut), c.bias)
    out_ref = tiled[r._where]
    r.close()
    idx = oracle.ref_index_calculation(c.x, c.centroid, None, None, nthreads=4).reshape(M, CB)
    acc, out = derive(idx, c.lut, c.bias, scale, lut_bias)
    assert np.array_equal(out.view(np.uint32), out_ref.view(np.uint32)), "numpy derivation != reference operator"
    mapping = {k: np.uint32(cfg[k]) for k in ("loop_order", "load_type", "n_stile", "f_stile", "n_mtile", "f_mtile",
                                               "cb_mtile", "f_load", "cb_load")}
    np.savez_compressed(os.path.join(OUT, name + ".npz"), x=c.x, centroid=c.centroid, lut=c.lut, bias=c.bias,
                        scale=np.float32(scale), lut_bias=np.float32(lut_bias), idx=idx, acc=acc, out=out,
                        out_ref=out_ref, out_ref_tiled=tiled, **mapping)
    print(f"{name}: reference operator {case_name} M={M} N={N} CB={CB} CT={CT} v={v}: bit-identical to derivation")


def main():
    assert oracle.have_reference(), "oracle/_ref is missing: run `make -C oracle` with the reference tree mounted"
    cases = [
        ("normal_v2_ct16", dict(M=48, K=64, N=64, v=2, CT=16, seed=11)),
        ("normal_v4_ct8", dict(M=40, K=64, N=48, v=4, CT=8, seed=12)),
        ("normal_v8_ct32", dict(M=33, K=128, N=32, v=8, CT=32, seed=13)),
        ("normal_v1_ct5", dict(M=17, K=24, N=16, v=1, CT=5, seed=14)),
        ("normal_v3_ct64", dict(M=9, K=48, N=80, v=3, CT=64, seed=15)),
    ]
    for name, kw in cases:
        c = synth.make_case(**kw)
        emit(name, c.x, c.centroid, c.lut, c.bias, c.scale, c.lut_bias)
    c = synth.make_case(M=32, K=64, N=64, v=2, CT=16, seed=21, scale=0.1, lut_bias=0.2, reference_style=True)
    emit("reference_style_v2_ct16", c.x, c.centroid, c.lut, c.bias, c.scale, c.lut_bias)
    c = synth.make_case(M=64, K=64, N=64, v=2, CT=16, seed=22)
    emit("tiled_v2_ct16", c.x, c.centroid, c.lut, c.bias, c.scale, c.lut_bias, n_stile=16, cb_mtile=8)
    for name, v, CT, seed in (("adversarial_v2_ct16", 2, 16, 31), ("adversarial_v4_ct8", 4, 8, 32)):
        CB, M, N = 32, 64, 32
        x, cent = adversarial(M, CB, CT, v, seed)
        w = synth.make_case(M=1, K=CB * v, N=N, v=v, CT=CT, seed=seed)
        emit(name, x, cent, w.lut, w.bias, w.scale, 0.0)
    # NaN / Inf rows: comparisons with NaN are false, so the earlier index is kept
    c = synth.make_case(M=8, K=32, N=16, v=2, CT=8, seed=41)
    c.x[0, :4] = np.nan
    c.x[1, 4:8] = np.inf
    c.x[2, 8:10] = -np.inf
    c.centroid[3, 2, 0] = np.nan
    emit("nonfinite_v2_ct8", c.x, c.centroid, c.lut, c.bias, c.scale, c.lut_bias)
    # the reference's whole operator (host code + DPU kernel), three loop-order / load-type corners
    assert oracle.have_ref_amm(), "oracle/_ref/libref_amm_host.so is missing"
    emit_refamm("refamm_ncf_coarse", "small_NCF_l2", 51, 0.1, 0.2, reference_style=True)
    emit_refamm("refamm_fnc_static", "small_FNC_l0", 52, 0.013, -0.4)
    emit_refamm("refamm_cfn_fine", "small_CFN_l1", 53, 0.05, 0.0)


if __name__ == "__main__":
    main()
