"""The reference's whole operator - amm_host.cpp, index_calc_host.cpp, pim_lut_host.cpp and the DPU
kernel src/dpu/pim_lut_kernel.c, compiled unmodified onto the functional UPMEM stand-in of
oracle/upmem_shim - against the CPU restatement and the committed golden vectors.  This pins the
restatement's LUT gather-accumulate and dequantisation to the reference's own code, for every loop
order and LUT load type the DPU kernel has."""
import numpy as np
import pytest

import oracle
from conftest import golden_names, load_golden
from pim_dl_asplos_b200 import synth

needs_ref = pytest.mark.skipif(not oracle.have_ref_amm(), reason="oracle/_ref (built from the reference tree) absent")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def run_case(name, seed, scale, lut_bias, **kw):
    cfg = oracle.REF_AMM_CASES[name]
    c = synth.make_case(M=cfg["M"], K=cfg["CB"] * cfg["v"], N=cfg["N"], v=cfg["v"], CT=cfg["CT"], seed=seed,
                        scale=scale, lut_bias=lut_bias, **kw)
    r = oracle.ref_amm_case(name, scale=scale, lut_bias=lut_bias, nthreads=4)
    try:
        got = r(c.x, c.centroid, c.lut, c.bias)
        again = r(c.x, c.centroid, c.lut, c.bias)   # MRAM persists between launches, as on the device
    finally:
        r.close()
    want, _, _ = oracle.amm(c.x, c.centroid, c.lut, c.bias, scale, lut_bias)
    assert np.array_equal(bits(got), bits(want)), f"{name}: restatement differs from the reference operator"
    assert np.array_equal(bits(again), bits(want)), f"{name}: second launch differs"


@needs_ref
@pytest.mark.parametrize("loop_order", range(6))
@pytest.mark.parametrize("load_type", range(3))
def test_every_loop_order_and_load_type(loop_order, load_type):
    run_case("small_%s_l%d" % (oracle.LOOP_ORDERS[loop_order], load_type), 100 + loop_order * 3 + load_type, 0.037, 0.21)


@needs_ref
@pytest.mark.parametrize("name,kw", [("example_like", dict(reference_style=True)), ("bert_base_proj", {}),
                                     ("bert_base_proj_static", {})])
def test_larger_mappings(name, kw):
    run_case(name, 7, 0.1, 0.2, **kw)


@needs_ref
def test_saturated_tables_and_ties():
    """Extreme table values (+127 / -128 everywhere) and exact distance ties through the reference operator."""
    name = "small_NCF_l2"
    cfg = oracle.REF_AMM_CASES[name]
    M, N, CB, CT, v = (cfg[k] for k in ("M", "N", "CB", "CT", "v"))
    rng = np.random.default_rng(5)
    x = (rng.integers(-8, 9, (M, CB * v)) * 0.125).astype(np.float32)
    cent = (rng.integers(-4, 5, (CB, CT, v)) * 0.25).astype(np.float32)
    cent[:, CT - 1] = cent[:, 0]      # duplicate centroids: the lower index must win
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    r = oracle.ref_amm_case(name, scale=0.5, lut_bias=0.0, nthreads=2)
    try:
        for fill in (127, -128):
            lut = np.full((CB, CT, N), fill, dtype=np.int8)
            got = r(x, cent, lut, bias)
            want, idx, acc = oracle.amm(x, cent, lut, bias, 0.5, 0.0)
            assert (acc == fill * CB).all() and (idx != CT - 1).all()
            assert np.array_equal(bits(got), bits(want))
    finally:
        r.close()


@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith("refamm_")])
def test_golden_reference_operator_outputs(name):
    """Runs without the reference tree: the committed outputs of the reference operator."""
    g = load_golden(name)
    out, idx, acc = oracle.amm(g["x"], g["centroid"], g["lut"], g["bias"], float(g["scale"]), float(g["lut_bias"]))
    assert np.array_equal(bits(out), bits(g["out_ref"]))
    M, N = out.shape
    lut_par = N // int(g["f_stile"])
    offs = np.array([[oracle.tiled_output_offset(i, j, int(g["n_stile"]), int(g["f_stile"]), int(g["f_mtile"]), lut_par)
                      for j in range(N)] for i in range(M)])
    assert np.array_equal(bits(g["out_ref_tiled"][offs.ravel()]), bits(out.ravel()))


@needs_ref
def test_stand_in_rejects_a_short_read():
    """The stand-in's own error path: reading a symbol that was never written fails the DPU_ASSERT-style check."""
    import ctypes
    L = ctypes.CDLL(oracle._REF_AMM_PATH)

    class Set(ctypes.Structure):
        _fields_ = [("impl", ctypes.c_void_p), ("single", ctypes.c_int32)]

    s = Set()
    L.dpu_alloc.argtypes = [ctypes.c_uint32, ctypes.c_char_p, ctypes.POINTER(Set)]
    assert L.dpu_alloc(2, None, ctypes.byref(s)) == 0
    L.shim_nth.restype = Set
    L.shim_nth.argtypes = [Set, ctypes.c_uint32]
    buf = (ctypes.c_int32 * 4)()
    L.dpu_prepare_xfer.argtypes = [Set, ctypes.c_void_p]
    assert L.dpu_prepare_xfer(L.shim_nth(s, 0), buf) == 0
    L.dpu_push_xfer.argtypes = [Set, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_size_t, ctypes.c_int]
    assert L.dpu_push_xfer(s, 1, b"output_data", 0, 16, 0) != 0      # FROM_DPU before anything was produced
    L.dpu_launch.argtypes = [Set, ctypes.c_int]
    assert L.dpu_launch(s, 0) != 0                                     # no program loaded
    L.dpu_free.argtypes = [Set]
    assert L.dpu_free(s) == 0


needs_ref_cpu = pytest.mark.skipif(not oracle.have_ref_amm_cpu(), reason="oracle/_ref/libref_amm_cpu.so absent")


@needs_ref_cpu
@pytest.mark.parametrize("M,K,N,v,CT", [(64, 128, 96, 2, 16), (33, 96, 48, 4, 8), (17, 30, 16, 3, 5), (128, 256, 64, 8, 32)])
def test_restatement_equals_reference_amm_cpu(M, K, N, v, CT):
    """amm_cpu() of the reference's test_amm.cpp, compiled unmodified: the reference's own CPU path."""
    c = synth.make_case(M=M, K=K, N=N, v=v, CT=CT, seed=M + N)
    got = oracle.ref_amm_cpu(c.x, c.centroid, c.lut, c.bias, c.scale, 0.0, nthreads=4)
    want, idx, acc = oracle.amm(c.x, c.centroid, c.lut, c.bias, c.scale, 0.0)
    assert np.array_equal(bits(got), bits(want))
    # with a LUT bias the reference's checker adds it once, the production path CB times: the known
    # inconsistency, restated by dequant_checker_variant
    got_b = oracle.ref_amm_cpu(c.x, c.centroid, c.lut, c.bias, c.scale, 0.2, nthreads=4)
    assert np.array_equal(bits(got_b), bits(oracle.dequant_checker_variant(acc, c.bias, c.scale, 0.2)))


@needs_ref_cpu
@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith(("adversarial", "nonfinite", "normal_v2"))])
def test_reference_amm_cpu_on_golden_vectors(name):
    g = load_golden(name)
    if float(g["lut_bias"]) != 0.0:
        pytest.skip("checker variant differs by design when the LUT bias is not zero")
    got = oracle.ref_amm_cpu(g["x"], g["centroid"], g["lut"], g["bias"], float(g["scale"]), 0.0, nthreads=2)
    finite = np.isfinite(g["out"])
    assert np.array_equal(bits(got)[finite], bits(g["out"])[finite])
