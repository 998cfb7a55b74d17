"""CPU oracle for the LUT-NN approximate matrix multiply (AMM).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and the timed CPU baseline.
Only tests, the smoke check and the benchmark's CPU-baseline legs may import this
package; the shipped library never does.

Two layers live here:

* ``liblutamm_oracle.so`` - the plain-C restatement (``lutamm_oracle.c``), fast enough
  for the full benchmark shapes, OpenMP over tokens;
* ``_ref/libref_index_calc.so`` - the reference's own, unmodified
  ``inference-engine/src/host/index_calc_host.cpp`` behind a C-linkage shim, built by
  the Makefile when the reference tree is present.  It pins the closest-centroid
  search of the restatement bit for bit.

* ``_ref/libref_amm_host.so`` + ``_ref/dpu_kernel_*.so`` - the reference's whole AMM
  (``amm_host.cpp``, ``index_calc_host.cpp``, ``pim_lut_host.cpp`` and the DPU kernel
  ``src/dpu/pim_lut_kernel.c``, all unmodified) running on host threads through the
  functional UPMEM stand-in in ``upmem_shim/``.  It pins the LUT gather-accumulate and
  the dequantisation of the restatement against the reference's own code
  (`RefAmm`, `build_ref_kernel`).

* ``_ref/libref_amm_cpu.so`` - the reference's own CPU statement of the whole operator,
  ``amm_cpu()`` of ``inference-engine/test/test_amm.cpp`` (that file compiled unmodified,
  its ``main`` renamed): the second opinion on the restatement and the timed CPU baseline
  (`ref_amm_cpu`).

A third, numpy-only statement of the search (`numpy_index_calculation`) exists so the
C restatement is cross-checked by an independent implementation on small cases.

Parity status: closest-centroid search pinned against the unmodified reference source
and the committed golden vectors generated from it; gather-accumulate and dequantisation
(``pim_lut_host.cpp:201``, restated operation by operation) pinned bit for bit against the
unmodified reference operator on the UPMEM stand-in, for all six loop orders and three LUT
load types of the DPU kernel.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liblutamm_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libref_index_calc.so")
_REF_AMM_PATH = os.path.join(_HERE, "_ref", "libref_amm_host.so")
_REF_AMM_CPU_PATH = os.path.join(_HERE, "_ref", "libref_amm_cpu.so")
# The reference tree (needed only to rebuild oracle/_ref): $LUTAMM_REFERENCE_DIR, else a checkout named
# `reference` beside this repository.
_REF_TREE = os.environ.get("LUTAMM_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")

_u32 = ctypes.c_uint32
_fp = ctypes.POINTER(ctypes.c_float)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_i8p = ctypes.POINTER(ctypes.c_int8)
_i32p = ctypes.POINTER(ctypes.c_int32)


def build(force: bool = False) -> None:
    """Compile the C restatement (and the reference object when its tree is present)."""
    need = force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "lutamm_oracle.c")))
    if need or (have_reference_tree() and not (os.path.exists(_REF_PATH) and os.path.exists(_REF_AMM_PATH)
                                               and os.path.exists(_REF_AMM_CPU_PATH))):
        subprocess.run(["make", "-C", _HERE, "all", "REF=" + _REF_TREE], check=True, stdout=subprocess.DEVNULL)
    if have_reference_tree():
        build_ref_cases()


def have_reference_tree() -> bool:
    return os.path.exists(os.path.join(_REF_TREE, "inference-engine/src/host/index_calc_host.cpp"))


_lib = None
_ref = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        L.oracle_index_calculation.argtypes = [_fp, _fp, _u16p, _u32, _u32, _u32, _u32, _u32, ctypes.c_int]
        L.oracle_index_calculation.restype = None
        L.oracle_index_calculation_tiled.argtypes = [_fp, _fp, _u16p, _u32, _u32, _u32, _u32, _u32, _u32, _u32, ctypes.c_int]
        L.oracle_index_calculation_tiled.restype = None
        L.oracle_lut_gather.argtypes = [_u16p, _i8p, _i32p, _u32, _u32, _u32, _u32, ctypes.c_int]
        L.oracle_lut_gather.restype = None
        L.oracle_dequant.argtypes = [_i32p, _fp, _fp, _u32, _u32, _u32, ctypes.c_float, ctypes.c_float, ctypes.c_int]
        L.oracle_dequant.restype = None
        L.oracle_dequant_checker_variant.argtypes = [_i32p, _fp, _fp, _u32, _u32, ctypes.c_float, ctypes.c_float, ctypes.c_int]
        L.oracle_dequant_checker_variant.restype = None
        L.oracle_amm.argtypes = [_fp, _fp, _i8p, _fp, _fp, _u16p, _i32p, _u32, _u32, _u32, _u32, _u32, _u32,
                                 ctypes.c_float, ctypes.c_float, ctypes.c_int]
        L.oracle_amm.restype = None
        L.oracle_tiled_output_offset.argtypes = [_u32] * 6
        L.oracle_tiled_output_offset.restype = ctypes.c_uint64
        L.oracle_reorder_lut.argtypes = [_i8p, _i8p, _u32, _u32, _u32, _u32]
        L.oracle_reorder_lut.restype = None
        _lib = L
    return _lib


def have_reference() -> bool:
    return os.path.exists(_REF_PATH)


def ref() -> ctypes.CDLL:
    """The reference's own index_calculation (unmodified source) behind ref_shim.cpp."""
    global _ref
    if _ref is None:
        R = ctypes.CDLL(_REF_PATH)
        R.ref_index_calculation.argtypes = [_fp, _fp, _u16p] + [_u32] * 8
        R.ref_index_calculation.restype = None
        _ref = R
    return _ref


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def default_threads() -> int:
    return os.cpu_count() or 1


def _chk(x, centroid):
    x = np.ascontiguousarray(x, dtype=np.float32)
    centroid = np.ascontiguousarray(centroid, dtype=np.float32)
    assert x.ndim == 2 and centroid.ndim == 3
    M, K = x.shape
    CB, CT, v = centroid.shape
    assert CB * v == K, "input_feature_len must equal num_codebook * sub_vec_len"
    return x, centroid, M, K, CB, CT, v


def index_calculation(x, centroid, nthreads: int | None = None) -> np.ndarray:
    """uint16 idx[M][CB] by the C restatement."""
    x, centroid, M, K, CB, CT, v = _chk(x, centroid)
    idx = np.zeros((M, CB), dtype=np.uint16)
    if M and CB:
        lib().oracle_index_calculation(_p(x, _fp), _p(centroid, _fp), _p(idx, _u16p), M, K, v, CB, CT,
                                       nthreads or default_threads())
    return idx


def index_calculation_tiled(x, centroid, n_stile: int, cb_mtile: int, nthreads: int | None = None) -> np.ndarray:
    """Flat uint16 index buffer in the reference's tiled layout (index_calc_host.cpp:41-49)."""
    x, centroid, M, K, CB, CT, v = _chk(x, centroid)
    idx = np.zeros(M * CB, dtype=np.uint16)
    lib().oracle_index_calculation_tiled(_p(x, _fp), _p(centroid, _fp), _p(idx, _u16p), M, K, v, CB, CT,
                                         n_stile, cb_mtile, nthreads or default_threads())
    return idx


def ref_index_calculation(x, centroid, n_stile: int | None = None, cb_mtile: int | None = None,
                          nthreads: int | None = None) -> np.ndarray:
    """Flat uint16 buffer straight from the reference object; row-major [M][CB] by default."""
    x, centroid, M, K, CB, CT, v = _chk(x, centroid)
    idx = np.zeros(M * CB, dtype=np.uint16)
    ref().ref_index_calculation(_p(x, _fp), _p(centroid, _fp), _p(idx, _u16p), M, K, v, CB, CT,
                                nthreads or default_threads(), n_stile or M, cb_mtile or CB)
    return idx


def untile_index(flat: np.ndarray, M: int, CB: int, n_stile: int, cb_mtile: int) -> np.ndarray:
    """Tiled [n_tile][cb_tile][n_in][cb_in] -> row-major [M][CB]."""
    t = flat.reshape(M // n_stile, CB // cb_mtile, n_stile, cb_mtile)
    return np.ascontiguousarray(t.transpose(0, 2, 1, 3)).reshape(M, CB)


def lut_gather(idx, lut, nthreads: int | None = None) -> np.ndarray:
    idx = np.ascontiguousarray(idx, dtype=np.uint16)
    lut = np.ascontiguousarray(lut, dtype=np.int8)
    M, CB = idx.shape
    CB2, CT, N = lut.shape
    assert CB == CB2
    acc = np.zeros((M, N), dtype=np.int32)
    if M and N:
        lib().oracle_lut_gather(_p(idx, _u16p), _p(lut, _i8p), _p(acc, _i32p), M, CB, CT, N,
                                nthreads or default_threads())
    return acc


def dequant(acc, bias, CB: int, scale: float, lut_bias: float = 0.0, nthreads: int | None = None) -> np.ndarray:
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    M, N = acc.shape
    out = np.zeros((M, N), dtype=np.float32)
    if M and N:
        lib().oracle_dequant(_p(acc, _i32p), _p(bias, _fp), _p(out, _fp), M, N, CB, scale, lut_bias,
                             nthreads or default_threads())
    return out


def dequant_checker_variant(acc, bias, scale: float, lut_bias: float = 0.0) -> np.ndarray:
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    M, N = acc.shape
    out = np.zeros((M, N), dtype=np.float32)
    lib().oracle_dequant_checker_variant(_p(acc, _i32p), _p(bias, _fp), _p(out, _fp), M, N, scale, lut_bias,
                                         default_threads())
    return out


def amm(x, centroid, lut, bias, scale: float, lut_bias: float = 0.0, nthreads: int | None = None):
    """Whole operator.  Returns (out fp32 [M][N], idx uint16 [M][CB], acc int32 [M][N])."""
    x, centroid, M, K, CB, CT, v = _chk(x, centroid)
    lut = np.ascontiguousarray(lut, dtype=np.int8)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    N = lut.shape[2]
    assert lut.shape[:2] == (CB, CT) and bias.shape == (N,)
    out = np.zeros((M, N), dtype=np.float32)
    idx = np.zeros((M, CB), dtype=np.uint16)
    acc = np.zeros((M, N), dtype=np.int32)
    if M:
        lib().oracle_amm(_p(x, _fp), _p(centroid, _fp), _p(lut, _i8p), _p(bias, _fp), _p(out, _fp),
                         _p(idx, _u16p), _p(acc, _i32p), M, K, v, CB, CT, N, scale, lut_bias,
                         nthreads or default_threads())
    return out, idx, acc


def gelu_tanh(y: np.ndarray, through_f16: bool = False) -> np.ndarray:
    """Checker for the activation the library can fuse after the dequantisation.  The reference
    applies GELU to the FFN1 output as a separate pass (inference-engine/src/host/transformer_layer.cpp:503,
    ggml_gelu_inplace).  ggml is an un-vendored submodule without a recoverable commit, so this follows
    its published definition instead of its source - 0.5 x (1 + tanh(sqrt(2/pi) x (1 + 0.044715 x^2))),
    evaluated per fp16 value through a table when `through_f16` (input rounded to fp16, result rounded to
    fp16) - and is evaluated in float64 here: parity unpinned, compared within a stated tolerance."""
    x = np.asarray(y, dtype=np.float32)
    if through_f16:
        x = x.astype(np.float16).astype(np.float32)
    xd = x.astype(np.float64)
    g = 0.5 * xd * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * xd * (1.0 + 0.044715 * xd * xd)))
    g = g.astype(np.float32)
    if through_f16:
        g = g.astype(np.float16).astype(np.float32)
    return g


def tiled_output_offset(i: int, j: int, n_stile: int, f_stile: int, f_mtile: int, lut_parallelism: int) -> int:
    return int(lib().oracle_tiled_output_offset(i, j, n_stile, f_stile, f_mtile, lut_parallelism))


def reorder_lut(lut: np.ndarray, tile: int) -> np.ndarray:
    lut = np.ascontiguousarray(lut, dtype=np.int8)
    CB, CT, N = lut.shape
    out = np.zeros(CB * CT * N, dtype=np.int8)
    lib().oracle_reorder_lut(_p(lut, _i8p), _p(out, _i8p), CB, CT, N, tile)
    return out


# ---------------------------------------------------------------------------------------
# Independent numpy statement of the search, for cross-checking the C code on small cases.
# ---------------------------------------------------------------------------------------
def numpy_index_calculation(x, centroid) -> np.ndarray:
    """index_calc_host.cpp:11-40 in numpy: fp32 ops one at a time (numpy never fuses),
    dimension-ordered accumulation, sequential hysteresis scan over the centroids."""
    x, centroid, M, K, CB, CT, v = _chk(x, centroid)
    xs = x.reshape(M, CB, 1, v)
    dist = np.zeros((M, CB, CT), dtype=np.float32)
    for d in range(v):
        e = (xs[..., d] - centroid[None, :, :, d]).astype(np.float32)
        sq = (e * e).astype(np.float32)
        dist = (dist + sq).astype(np.float32)
    mn = dist[..., 0].copy()
    best = np.zeros((M, CB), dtype=np.uint16)
    eps = np.float64(1e-6)
    for c in range(1, CT):
        with np.errstate(invalid="ignore"):
            diff = (mn - dist[..., c]).astype(np.float32)
            take = diff.astype(np.float64) > eps
        mn = np.where(take, dist[..., c], mn)
        best = np.where(take, np.uint16(c), best)
    return best


# ---------------------------------------------------------------------------------------
# The reference's whole AMM on the UPMEM stand-in (upmem_shim/): unmodified reference code.
# ---------------------------------------------------------------------------------------
class RefIndexCalcParams(ctypes.Structure):
    """The reference's IndexCalcParams, field for field (src/host/defines.h:12-24)."""
    _fields_ = [(n, _u32) for n in ("n", "input_feature_len", "sub_vec_len", "num_codebook", "num_centroid",
                                    "num_threads", "n_stile_size", "cb_mtile_size")]


class RefLUTParams(ctypes.Structure):
    """The reference's LUTParams, field for field (src/host/defines.h:26-50)."""
    _fields_ = [("n", _u32), ("output_feature_len", _u32), ("num_codebook", _u32), ("num_centroid", _u32),
                ("scale", ctypes.c_float), ("bias", ctypes.c_float), ("num_threads", _u32), ("dpu_num", _u32),
                ("input_parallelism", _u32), ("lut_parallelism", _u32), ("feature_stile_size", _u32),
                ("n_stile_size", _u32), ("n_mtile_size", _u32), ("feature_mtile_size", _u32),
                ("cb_mtile_size", _u32), ("lut_load_type", _u32), ("feature_load_tile_size", _u32),
                ("cb_load_tile_size", _u32)]


LOOP_ORDERS = ("NFC", "NCF", "FNC", "FCN", "CNF", "CFN")   # src/dpu/CMakeLists.txt:28-40
LOAD_STATIC, LOAD_FINE_GRAIN, LOAD_COARSE_GRAIN = 0, 1, 2  # enum LUTLoadType, src/host/defines.h:10


def ref_kernel_path(CB, CT, loop_order, load_type, n_stile, f_stile, n_mtile, f_mtile, cb_mtile, f_load, cb_load,
                    nr_tasklets=16) -> str:
    name = "dpu_kernel_cb%d_ct%d_%s_l%d_s%dx%d_m%dx%dx%d_t%dx%d_k%d.so" % (
        CB, CT, LOOP_ORDERS[loop_order], load_type, n_stile, f_stile, n_mtile, f_mtile, cb_mtile, f_load, cb_load,
        nr_tasklets)
    return os.path.join(_HERE, "_ref", name)


def build_ref_kernel(CB, CT, loop_order, load_type, n_stile, f_stile, n_mtile, f_mtile, cb_mtile, f_load, cb_load,
                     nr_tasklets=16) -> str:
    """Compile the reference's DPU kernel for one configuration (the -D list of src/dpu/CMakeLists.txt:20-60)
    into a host shared object; returns its path.  A prebuilt object is reused."""
    out = ref_kernel_path(CB, CT, loop_order, load_type, n_stile, f_stile, n_mtile, f_mtile, cb_mtile, f_load,
                          cb_load, nr_tasklets)
    if os.path.exists(out):
        return out
    if not have_reference_tree():
        raise FileNotFoundError("reference tree absent and %s was not prebuilt" % os.path.basename(out))
    defs = ["-DNR_TASKLETS=%d" % nr_tasklets, "-DNUM_CODEBOOK=%d" % CB, "-DNUM_CENTROID=%d" % CT,
            "-DLOOP_ORDER_" + LOOP_ORDERS[loop_order],
            "-DN_STILE_SIZE=%d" % n_stile, "-DFEATURE_STILE_SIZE=%d" % f_stile,
            "-DN_MTILE_SIZE=%d" % n_mtile, "-DFEATURE_MTILE_SIZE=%d" % f_mtile, "-DCB_MTILE_SIZE=%d" % cb_mtile,
            "-DFEATURE_LOAD_TILE_SIZE=%d" % f_load, "-DCB_LOAD_TILE_SIZE=%d" % cb_load]
    if load_type == LOAD_STATIC:
        defs.append("-DSTATIC_LUT_TABLE")
    elif load_type == LOAD_FINE_GRAIN:
        defs.append("-DFINE_GRAIN")
    subprocess.run(["make", "-C", _HERE, "ref_kernel", "REF=" + _REF_TREE, "KOUT=" + out, "KDEFS=" + " ".join(defs)],
                   check=True, stdout=subprocess.DEVNULL)
    return out


def have_ref_amm() -> bool:
    return os.path.exists(_REF_AMM_PATH)


_ref_amm = None


def _ref_amm_lib() -> ctypes.CDLL:
    global _ref_amm
    if _ref_amm is None:
        R = ctypes.CDLL(_REF_AMM_PATH)
        R.ref_amm_open.argtypes = [_u32, ctypes.c_char_p]
        R.ref_amm_open.restype = ctypes.c_void_p
        R.ref_amm_run.argtypes = [ctypes.c_void_p, _fp, _fp, _i8p, _fp, _fp,
                                  ctypes.POINTER(RefIndexCalcParams), ctypes.POINTER(RefLUTParams)]
        R.ref_amm_run.restype = None
        R.ref_amm_close.argtypes = [ctypes.c_void_p]
        R.ref_amm_close.restype = None
        _ref_amm = R
    return _ref_amm


class RefAmm:
    """One AMM operator of the reference, run by the reference's own amm_host() and DPU kernel.

    The mapping parameters are those of the reference's YAML (`lut_params`, config/amm.yaml):
    the token axis is cut into `input_parallelism` = M / n_stile blocks, the output features
    into `lut_parallelism` = N / f_stile blocks, one DPU per (token block, feature block).
    """

    def __init__(self, M, N, CB, CT, v, *, loop_order=0, load_type=LOAD_COARSE_GRAIN, n_stile, f_stile, n_mtile,
                 f_mtile, cb_mtile, f_load, cb_load, nr_tasklets=16, scale=1.0, lut_bias=0.0, nthreads=None):
        assert M % n_stile == 0 and N % f_stile == 0
        self.M, self.N, self.CB, self.CT, self.v = M, N, CB, CT, v
        self.load_type = load_type
        nthreads = nthreads or default_threads()
        ip_par, lut_par = M // n_stile, N // f_stile
        self.ip = RefIndexCalcParams(M, CB * v, v, CB, CT, nthreads, n_stile, cb_mtile)
        self.lp = RefLUTParams(M, N, CB, CT, scale, lut_bias, nthreads, ip_par * lut_par, ip_par, lut_par,
                               f_stile, n_stile, n_mtile, f_mtile, cb_mtile, load_type, f_load, cb_load)
        kernel = build_ref_kernel(CB, CT, loop_order, load_type, n_stile, f_stile, n_mtile, f_mtile, cb_mtile,
                                  f_load, cb_load, nr_tasklets)
        self._h = _ref_amm_lib().ref_amm_open(ip_par * lut_par, kernel.encode())
        # output position of element (i, j) in the DPU-tiled result (test/test_amm.cpp:193-202)
        i = np.arange(M, dtype=np.int64)[:, None]
        j = np.arange(N, dtype=np.int64)[None, :]
        dpu = (i // n_stile) * lut_par + j // f_stile
        jd = j % f_stile
        self._where = (dpu * n_stile * f_stile + (jd // f_mtile) * n_stile * f_mtile
                       + (i % n_stile) * f_mtile + jd % f_mtile)

    def dpu_lut(self, lut: np.ndarray) -> np.ndarray:
        """Canonical [CB][CT][N] table -> the DPU layout of reorder_pim_lut (test/test_amm.cpp:71-121)."""
        tile = self.lp.feature_stile_size if self.load_type == LOAD_STATIC else self.lp.feature_load_tile_size
        return reorder_lut(lut, tile)

    def run_tiled(self, x, centroid, lut_dpu, bias) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        centroid = np.ascontiguousarray(centroid, dtype=np.float32)
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        assert x.shape == (self.M, self.CB * self.v) and centroid.shape == (self.CB, self.CT, self.v)
        assert lut_dpu.dtype == np.int8 and lut_dpu.size == self.CB * self.CT * self.N and bias.size == self.N
        out = np.empty(self.M * self.N, dtype=np.float32)
        _ref_amm_lib().ref_amm_run(self._h, _p(x, _fp), _p(centroid, _fp), _p(lut_dpu, _i8p), _p(bias, _fp),
                                   _p(out, _fp), ctypes.byref(self.ip), ctypes.byref(self.lp))
        return out

    def __call__(self, x, centroid, lut, bias) -> np.ndarray:
        """Canonical tensors in, row-major [M][N] fp32 out."""
        return self.run_tiled(x, centroid, self.dpu_lut(lut), bias)[self._where]

    def close(self):
        if self._h:
            _ref_amm_lib().ref_amm_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _small(lo, lt):
    return dict(M=64, N=64, CB=16, CT=16, v=4, loop_order=lo, load_type=lt, n_stile=32, f_stile=32, n_mtile=16,
                f_mtile=16, cb_mtile=8, f_load=8, cb_load=4)


# The operator mappings the tests run through the reference's own code.  `build()` compiles the
# DPU kernel of each while the reference tree is at hand, so the objects travel prebuilt.
REF_AMM_CASES = {("small_%s_l%d" % (LOOP_ORDERS[lo], lt)): _small(lo, lt) for lo in range(6) for lt in range(3)}
REF_AMM_CASES.update({
    # the shape family of the reference's single-kernel example (config/single_kernel_output_example.yaml), shrunk
    "example_like": dict(M=256, N=256, CB=64, CT=16, v=4, loop_order=1, load_type=LOAD_COARSE_GRAIN, n_stile=128,
                         f_stile=128, n_mtile=64, f_mtile=32, cb_mtile=32, f_load=8, cb_load=32),
    # a BERT-base projection (hidden 768, sub-vector 2, 16 centroids) on 12 DPUs
    "bert_base_proj": dict(M=512, N=768, CB=384, CT=16, v=2, loop_order=1, load_type=LOAD_COARSE_GRAIN, n_stile=256,
                           f_stile=128, n_mtile=64, f_mtile=32, cb_mtile=128, f_load=8, cb_load=128),
    "bert_base_proj_static": dict(M=256, N=768, CB=384, CT=16, v=2, loop_order=0, load_type=LOAD_STATIC, n_stile=128,
                                  f_stile=8, n_mtile=64, f_mtile=8, cb_mtile=128, f_load=8, cb_load=128),
})


def ref_amm_case(name: str, **kw) -> RefAmm:
    c = dict(REF_AMM_CASES[name])
    return RefAmm(c.pop("M"), c.pop("N"), c.pop("CB"), c.pop("CT"), c.pop("v"), **c, **kw)


def build_ref_cases() -> None:
    for c in REF_AMM_CASES.values():
        build_ref_kernel(c["CB"], c["CT"], c["loop_order"], c["load_type"], c["n_stile"], c["f_stile"], c["n_mtile"],
                         c["f_mtile"], c["cb_mtile"], c["f_load"], c["cb_load"])


# ---------------------------------------------------------------------------------------
# Load-time table construction (model-calibration/pim_weight_converter.py:21-36, 83-91).
# ---------------------------------------------------------------------------------------
def build_lut(centroid, weight):
    """lut_f = bmm(centroid [CB][CT][v], weight.view(CB, v, N)) in fp32 with the sub-vector
    dimension accumulated in ascending order, one rounding per operation; then the converter's
    symmetric quantisation: scale = max|lut_f| / 127, lut = int8(rint(clip(lut_f / scale, -128, 127))),
    lut_bias = -scale * 0.  Returns (lut int8 [CB][CT][N], scale fp32, lut_bias fp32)."""
    centroid = np.ascontiguousarray(centroid, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    CB, CT, v = centroid.shape
    N = weight.shape[1]
    w = weight.reshape(CB, v, N)
    acc = np.zeros((CB, CT, N), dtype=np.float32)
    for d in range(v):
        acc = acc + centroid[:, :, d, None] * w[:, None, d, :]   # numpy fp32: multiply, then add, each rounded
    scale = np.float32(np.abs(acc).max()) / np.float32(127.0)
    if scale > 0:
        lut = np.rint(np.clip(acc / scale, np.float32(-128), np.float32(127))).astype(np.int8)
    else:
        lut = np.zeros((CB, CT, N), dtype=np.int8)
    return lut, np.float32(scale), np.float32(-scale * np.float32(0.0))


# ---------------------------------------------------------------------------------------
# The reference's own CPU AMM, amm_cpu() (test/test_amm.cpp:126-183), compiled unmodified.
# ---------------------------------------------------------------------------------------
def have_ref_amm_cpu() -> bool:
    return os.path.exists(_REF_AMM_CPU_PATH)


_ref_amm_cpu = None


def ref_amm_cpu(x, centroid, lut, bias, scale: float, lut_bias: float = 0.0, nthreads: int | None = None) -> np.ndarray:
    """Canonical tensors in, row-major [M][N] fp32 out.  Note that amm_cpu adds the LUT bias ONCE
    (test_amm.cpp:181) where the production path adds it num_codebook times (pim_lut_host.cpp:201);
    the two agree for lut_bias = 0, which converted weights always have."""
    global _ref_amm_cpu
    if _ref_amm_cpu is None:
        R = ctypes.CDLL(_REF_AMM_CPU_PATH)
        R.ref_amm_cpu.argtypes = [_fp, _fp, _i8p, _fp, _fp, ctypes.POINTER(RefIndexCalcParams), ctypes.POINTER(RefLUTParams)]
        R.ref_amm_cpu.restype = None
        _ref_amm_cpu = R
    x, centroid, M, K, CB, CT, v = _chk(x, centroid)
    lut = np.ascontiguousarray(lut, dtype=np.int8)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    N = lut.shape[2]
    t = nthreads or default_threads()
    ip = RefIndexCalcParams(M, K, v, CB, CT, t, max(M, 1), CB)
    lp = RefLUTParams(M, N, CB, CT, scale, lut_bias, t, 1, 1, 1, N, max(M, 1), max(M, 1), N, CB, 0, N, CB)
    out = np.empty((M, N), dtype=np.float32)
    _ref_amm_cpu.ref_amm_cpu(_p(x, _fp), _p(centroid, _fp), _p(lut, _i8p), _p(bias, _fp), _p(out, _fp),
                             ctypes.byref(ip), ctypes.byref(lp))
    return out
