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

A third, numpy-only statement of the search (`numpy_index_calculation`) exists so the
C restatement is cross-checked by an independent implementation on small cases.

Parity status: closest-centroid search pinned against the unmodified reference source
and the committed golden vectors generated from it; gather is exact integer addition;
dequantisation follows ``pim_lut_host.cpp:201`` operation by operation.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liblutamm_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libref_index_calc.so")

_u32 = ctypes.c_uint32
_fp = ctypes.POINTER(ctypes.c_float)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_i8p = ctypes.POINTER(ctypes.c_int8)
_i32p = ctypes.POINTER(ctypes.c_int32)


def build(force: bool = False) -> None:
    """Compile the C restatement (and the reference object when its tree is present)."""
    need = force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "lutamm_oracle.c")))
    ref_tree = os.path.exists("/root/reference/inference-engine/src/host/index_calc_host.cpp")
    if need or (ref_tree and not os.path.exists(_REF_PATH)):
        subprocess.run(["make", "-C", _HERE, "all"], check=True, stdout=subprocess.DEVNULL)


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
