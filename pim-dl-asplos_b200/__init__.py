"""B200-native LUT-NN approximate matrix multiply (AMM): Python host side.

This package is a thin mirror of the reference inference engine's operator interface
(inference-engine/src/host/amm_host.h:8-10, index_calc_host.h:5, pim_lut_host.h:14-15)
over the C ABI in include/lutamm.h.  All arithmetic happens in libpimdl_b200.so
(hand-written CUDA for sm_100a); there is no CPU or PyTorch implementation of the
operator here, and importing the compute entry points without the built library raises.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpimdl_b200.so")

OK, EINVAL, ECUDA, ENOLAYER, EUNSUPPORTED, EDEVICE, ENOMEM = 0, -1, -2, -3, -4, -5, -6
FLAG_ASYNC, FLAG_OUTPUT_TILED, FLAG_PEER_STORE = 1, 2, 4
VARIANT_AUTO, VARIANT_GATHER, VARIANT_UMMA = 0, 1, 2
INDEX_U8_ROWMAJOR, INDEX_U16_TILED = 0, 1
LUT_CANONICAL, LUT_DPU_TILED = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GELU_TANH_F16 = 0, 1, 2
EPILOGUE_AUTO, EPILOGUE_TRANSPOSE, EPILOGUE_COPY_ENGINE = 0, 1, 2

# every symbol include/lutamm.h declares
ABI_SYMBOLS = [
    "lutamm_create", "lutamm_destroy", "lutamm_set_stream", "lutamm_sync", "lutamm_last_error",
    "lutamm_version", "lutamm_load_weights", "lutamm_unload_weights", "lutamm_amm", "lutamm_amm_debug",
    "lutamm_index_calculation", "lutamm_pim_lut", "lutamm_set_plan", "lutamm_get_plan", "lutamm_set_activation", "lutamm_tune",
    "lutamm_enable_timing", "lutamm_get_timings", "lutamm_launch_count",
    "lutamm_amm_static_scratch", "lutamm_static_scratch_last_error", "lutamm_build_lut",
    "lutamm_load_weights_layout", "lutamm_measure_int8_peak",
    "lutamm_shard_unique_id", "lutamm_shard_init", "lutamm_shard_finalize", "lutamm_amm_column_sharded",
    "lutamm_amm_token_sharded", "lutamm_tune_sharding", "lutamm_plan_cache_save", "lutamm_plan_cache_load",
    "lutamm_selftest_bounded_wait", "lutamm_shard_alloc_gathered", "lutamm_shard_free_gathered",
]
SHARD_SEARCH_REPLICATED, SHARD_SEARCH_SPLIT = 0, 1
SHARD_ID_BYTES = 128


class LutAmmError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"lutamm error {code}: {msg}")
        self.code = code


class IndexCalcParams(ctypes.Structure):
    """Field-for-field the reference's IndexCalcParams (src/host/defines.h:12-24)."""
    _fields_ = [(n, ctypes.c_uint32) for n in (
        "n", "input_feature_len", "sub_vec_len", "num_codebook", "num_centroid", "num_threads",
        "n_stile_size", "cb_mtile_size")]


class LUTParams(ctypes.Structure):
    """Field-for-field the reference's LUTParams (src/host/defines.h:26-50)."""
    _fields_ = [("n", ctypes.c_uint32), ("output_feature_len", ctypes.c_uint32),
                ("num_codebook", ctypes.c_uint32), ("num_centroid", ctypes.c_uint32),
                ("scale", ctypes.c_float), ("bias", ctypes.c_float),
                ("num_threads", ctypes.c_uint32), ("dpu_num", ctypes.c_uint32),
                ("input_parallelism", ctypes.c_uint32), ("lut_parallelism", ctypes.c_uint32),
                ("feature_stile_size", ctypes.c_uint32), ("n_stile_size", ctypes.c_uint32),
                ("n_mtile_size", ctypes.c_uint32), ("feature_mtile_size", ctypes.c_uint32),
                ("cb_mtile_size", ctypes.c_uint32), ("lut_load_type", ctypes.c_uint32),
                ("feature_load_tile_size", ctypes.c_uint32), ("cb_load_tile_size", ctypes.c_uint32)]


class Plan(ctypes.Structure):
    _fields_ = [("variant", ctypes.c_uint32), ("ccs_tokens", ctypes.c_uint32), ("gather_cfg", ctypes.c_uint32),
                ("umma_n_tile", ctypes.c_uint32), ("umma_split", ctypes.c_uint32), ("umma_stages", ctypes.c_uint32),
                ("umma_groups", ctypes.c_uint32), ("umma_operand", ctypes.c_uint32),
                ("umma_sps", ctypes.c_uint32), ("umma_epilogue", ctypes.c_uint32)]

    def as_dict(self):
        return {k: getattr(self, k) for k in ("variant", "ccs_tokens", "gather_cfg", "umma_n_tile", "umma_split",
                                              "umma_stages", "umma_groups", "umma_operand", "umma_sps", "umma_epilogue")}


SHARDING_MODES = ("tokens_local", "tokens_gathered", "tokens_fused", "columns", "columns_split", "columns_fused")


class ShardingReport(ctypes.Structure):
    _fields_ = [("best", ctypes.c_uint32), ("world", ctypes.c_uint32), ("ms", ctypes.c_float * len(SHARDING_MODES))]


class Timings(ctypes.Structure):
    _fields_ = [("index_calc_ms", ctypes.c_float), ("lut_kernel_ms", ctypes.c_float),
                ("data_transfer_ms", ctypes.c_float), ("total_ms", ctypes.c_float)]


_lib = None


def load_library() -> ctypes.CDLL:
    """dlopen libpimdl_b200.so and type its entry points.  Raises if it has not been built:
    there is no fallback implementation."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(nvcc, sm_100a).  This package has no CPU fallback.")
    L = ctypes.CDLL(LIB_PATH)
    vp, u32, i32 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_int
    L.lutamm_version.restype = ctypes.c_char_p
    L.lutamm_version.argtypes = []
    L.lutamm_create.argtypes = [ctypes.POINTER(vp), i32]
    L.lutamm_destroy.argtypes = [vp]
    L.lutamm_set_stream.argtypes = [vp, vp]
    L.lutamm_sync.argtypes = [vp]
    L.lutamm_last_error.argtypes = [vp]
    L.lutamm_last_error.restype = ctypes.c_char_p
    L.lutamm_load_weights.argtypes = [vp, i32, vp, vp, vp, ctypes.POINTER(IndexCalcParams), ctypes.POINTER(LUTParams)]
    L.lutamm_load_weights_layout.argtypes = [vp, i32, vp, vp, vp, ctypes.POINTER(IndexCalcParams),
                                             ctypes.POINTER(LUTParams), u32]
    L.lutamm_unload_weights.argtypes = [vp, i32]
    L.lutamm_build_lut.argtypes = [vp, vp, vp, u32, u32, u32, u32, vp, ctypes.POINTER(ctypes.c_float),
                                   ctypes.POINTER(ctypes.c_float)]
    L.lutamm_amm.argtypes = [vp, i32, vp, vp, u32, u32]
    L.lutamm_amm_debug.argtypes = [vp, i32, vp, vp, u32, vp, vp, u32]
    L.lutamm_index_calculation.argtypes = [vp, i32, vp, vp, u32, u32]
    L.lutamm_pim_lut.argtypes = [vp, i32, vp, vp, u32, u32]
    L.lutamm_set_plan.argtypes = [vp, i32, ctypes.POINTER(Plan)]
    L.lutamm_get_plan.argtypes = [vp, i32, ctypes.POINTER(Plan)]
    L.lutamm_set_activation.argtypes = [vp, i32, u32]
    L.lutamm_tune.argtypes = [vp, i32, u32, ctypes.POINTER(Plan)]
    L.lutamm_enable_timing.argtypes = [vp, i32]
    L.lutamm_get_timings.argtypes = [vp, ctypes.POINTER(Timings)]
    L.lutamm_shard_unique_id.argtypes = [ctypes.c_char_p]
    L.lutamm_shard_init.argtypes = [vp, i32, i32, ctypes.c_char_p]
    L.lutamm_shard_finalize.argtypes = [vp]
    L.lutamm_amm_column_sharded.argtypes = [vp, i32, vp, vp, u32, u32, u32]
    L.lutamm_amm_token_sharded.argtypes = [vp, i32, vp, vp, u32, u32, u32]
    L.lutamm_tune_sharding.argtypes = [vp, i32, i32, u32, u32, ctypes.POINTER(ShardingReport)]
    L.lutamm_shard_alloc_gathered.argtypes = [vp, ctypes.c_size_t, ctypes.POINTER(vp)]
    L.lutamm_shard_free_gathered.argtypes = [vp, vp]
    L.lutamm_selftest_bounded_wait.argtypes = [vp, u32]
    L.lutamm_plan_cache_save.argtypes = [vp, ctypes.c_char_p]
    L.lutamm_plan_cache_load.argtypes = [vp, ctypes.c_char_p]
    dp = ctypes.POINTER(ctypes.c_double)
    L.lutamm_measure_int8_peak.argtypes = [vp, dp, dp, dp]
    L.lutamm_launch_count.argtypes = [vp]
    L.lutamm_launch_count.restype = ctypes.c_uint64
    L.lutamm_amm_static_scratch.argtypes = [i32, vp, vp, vp, vp, vp, vp, ctypes.POINTER(IndexCalcParams),
                                            ctypes.POINTER(LUTParams)]
    L.lutamm_static_scratch_last_error.argtypes = []
    L.lutamm_static_scratch_last_error.restype = ctypes.c_char_p
    for name in ABI_SYMBOLS:
        if name not in ("lutamm_version", "lutamm_last_error", "lutamm_launch_count", "lutamm_static_scratch_last_error"):
            getattr(L, name).restype = i32
    _lib = L
    return L


def _ptr(a) -> int:
    """Address of a numpy array (host) or of anything with data_ptr() (a torch tensor)."""
    if a is None:
        return 0
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"], "arrays handed to the C ABI must be contiguous"
        return a.ctypes.data
    if hasattr(a, "data_ptr"):
        assert a.is_contiguous(), "tensors handed to the C ABI must be contiguous"
        return a.data_ptr()
    return int(a)


def make_params(M: int, K: int, N: int, CB: int, CT: int, scale: float, lut_bias: float = 0.0, *,
                n_stile: int | None = None, f_stile: int | None = None, n_mtile: int | None = None,
                f_mtile: int | None = None, cb_mtile: int | None = None, num_threads: int = 1,
                lut_load_type: int = 0, f_load: int | None = None, cb_load: int | None = None):
    """Parameter blocks as parse_amm_configs() would fill them (src/host/parser.cpp:22-46).
    Tile sizes default to "one tile": the canonical row-major layouts."""
    n_stile = n_stile or max(M, 1)
    f_stile = f_stile or N
    n_mtile = n_mtile or n_stile
    f_mtile = f_mtile or f_stile
    cb_mtile = cb_mtile or CB
    ip = IndexCalcParams(M, K, K // CB, CB, CT, num_threads, n_stile, cb_mtile)
    lp = LUTParams()
    lp.n, lp.output_feature_len, lp.num_codebook, lp.num_centroid = M, N, CB, CT
    lp.scale, lp.bias = scale, lut_bias
    lp.num_threads = num_threads
    lp.input_parallelism = max(M // n_stile, 1)
    lp.lut_parallelism = max(N // f_stile, 1)
    lp.dpu_num = lp.input_parallelism * lp.lut_parallelism
    lp.feature_stile_size, lp.n_stile_size = f_stile, n_stile
    lp.n_mtile_size, lp.feature_mtile_size, lp.cb_mtile_size = n_mtile, f_mtile, cb_mtile
    lp.lut_load_type = lut_load_type
    lp.feature_load_tile_size, lp.cb_load_tile_size = f_load or f_mtile, cb_load or cb_mtile
    return ip, lp


@dataclass
class _LayerInfo:
    K: int
    N: int
    CB: int
    CT: int
    ip: IndexCalcParams = field(repr=False, default=None)
    lp: LUTParams = field(repr=False, default=None)


class LutAmmContext:
    """One context per process per GPU: the stand-in for the reference's dpu_set_t
    (allocate_dpu/free_dpu_set, src/host/dpu_common.h:11-38)."""

    def __init__(self, device: int = 0):
        self._L = load_library()
        h = ctypes.c_void_p()
        rc = self._L.lutamm_create(ctypes.byref(h), device)
        if rc != OK:
            raise LutAmmError(rc, self._L.lutamm_last_error(None).decode())
        self._h = h
        self.device = device
        self.layers: dict[int, _LayerInfo] = {}

    # -- plumbing
    def _check(self, rc: int):
        if rc != OK:
            raise LutAmmError(rc, self._L.lutamm_last_error(self._h).decode())

    def close(self):
        if getattr(self, "_h", None):
            self._L.lutamm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def set_stream(self, cuda_stream: int | None):
        self._check(self._L.lutamm_set_stream(self._h, cuda_stream or None))

    def sync(self):
        self._check(self._L.lutamm_sync(self._h))

    @property
    def launch_count(self) -> int:
        return int(self._L.lutamm_launch_count(self._h))

    # -- weights
    def load_weights(self, layer_id: int, centroid, lut, bias, scale: float, lut_bias: float = 0.0,
                     ip: IndexCalcParams | None = None, lp: LUTParams | None = None, lut_layout: int = LUT_CANONICAL):
        """centroid [CB][CT][v] fp32, lut [CB][CT][N] int8, bias [N] fp32 (numpy or torch).  With
        lut_layout=LUT_DPU_TILED `lut` is the flat table after the reference's reorder_pim_lut()
        (test/test_amm.cpp:71-121) and `lp` carries the tile sizes."""
        CB, CT, v = tuple(centroid.shape)
        N = int(lut.shape[2]) if lut_layout == LUT_CANONICAL else int(lp.output_feature_len)
        K = CB * v
        if ip is None or lp is None:
            ip, lp = make_params(0, K, N, CB, CT, scale, lut_bias)
        self._check(self._L.lutamm_load_weights_layout(self._h, layer_id, _ptr(centroid), _ptr(lut), _ptr(bias),
                                                       ctypes.byref(ip), ctypes.byref(lp), lut_layout))
        self.layers[layer_id] = _LayerInfo(K, N, CB, CT, ip, lp)

    def build_lut(self, centroid, weight, lut_out=None):
        """The table construction of the reference's converter (model-calibration/pim_weight_converter.py:21-36,
        83-91) on the GPU.  centroid [CB][CT][v] fp32, weight [CB*v][N] fp32 (numpy or torch, host or device);
        returns (lut int8 [CB][CT][N], scale, lut_bias)."""
        CB, CT, v = (int(d) for d in centroid.shape)
        K, N = (int(d) for d in weight.shape)
        if K != CB * v:
            raise ValueError("weight rows must equal num_codebook * sub_vec_len")
        if lut_out is None:
            lut_out = np.empty((CB, CT, N), dtype=np.int8)
        scale, lut_bias = ctypes.c_float(), ctypes.c_float()
        self._check(self._L.lutamm_build_lut(self._h, _ptr(centroid), _ptr(weight), CB, CT, v, N, _ptr(lut_out),
                                             ctypes.byref(scale), ctypes.byref(lut_bias)))
        return lut_out, float(scale.value), float(lut_bias.value)

    def unload_weights(self, layer_id: int):
        self._check(self._L.lutamm_unload_weights(self._h, layer_id))
        self.layers.pop(layer_id, None)

    # -- the operator (names follow the reference)
    def amm_host(self, layer_id: int, input_tensor, output_tensor, n_tokens: int | None = None, flags: int = 0):
        """amm_host() of the reference (src/host/amm_host.cpp:10-30)."""
        M = int(n_tokens if n_tokens is not None else input_tensor.shape[0])
        self._check(self._L.lutamm_amm(self._h, layer_id, _ptr(input_tensor), _ptr(output_tensor), M, flags))

    def amm_debug(self, layer_id: int, x: np.ndarray, flags: int = 0):
        """Host-array convenience for parity checks: returns (out fp32, idx uint8, acc int32)."""
        info = self.layers[layer_id]
        M = x.shape[0]
        out = np.zeros((M, info.N), dtype=np.float32)
        idx = np.zeros((M, info.CB), dtype=np.uint8)
        acc = np.zeros((M, info.N), dtype=np.int32)
        self._check(self._L.lutamm_amm_debug(self._h, layer_id, _ptr(x), _ptr(out), M, _ptr(idx), _ptr(acc), flags))
        return out, idx, acc

    def index_calculation(self, layer_id: int, input_tensor, index_out, n_tokens: int | None = None,
                          index_format: int = INDEX_U8_ROWMAJOR):
        """index_calculation() of the reference (src/host/index_calc_host.cpp:8-53)."""
        M = int(n_tokens if n_tokens is not None else input_tensor.shape[0])
        self._check(self._L.lutamm_index_calculation(self._h, layer_id, _ptr(input_tensor), _ptr(index_out), M,
                                                     index_format))

    def pim_lut(self, layer_id: int, input_index, output_tensor, n_tokens: int | None = None, flags: int = 0):
        """pim_lut() of the reference (src/host/pim_lut_host.cpp:121-222)."""
        M = int(n_tokens if n_tokens is not None else input_index.shape[0])
        self._check(self._L.lutamm_pim_lut(self._h, layer_id, _ptr(input_index), _ptr(output_tensor), M, flags))

    # -- one AMM across the GPUs of a box (one process per GPU)
    def shard_init(self, rank: int | None = None, world: int | None = None, group=None):
        """Join this context to an NCCL communicator of its own over `world` ranks.  The 128-byte id is made on
        rank 0 and broadcast through torch.distributed (any backend), which must be initialised."""
        import torch
        import torch.distributed as dist
        rank = dist.get_rank(group) if rank is None else rank
        world = dist.get_world_size(group) if world is None else world
        buf = ctypes.create_string_buffer(SHARD_ID_BYTES)
        if rank == 0:
            rc = self._L.lutamm_shard_unique_id(buf)
            if rc != OK:
                raise LutAmmError(rc, self._L.lutamm_last_error(None).decode())
        dev = torch.device("cuda", self.device) if dist.get_backend(group) == "nccl" else torch.device("cpu")
        t = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).to(dev)
        dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        self._check(self._L.lutamm_shard_init(self._h, rank, world, bytes(t.cpu().numpy().tobytes())))
        self.rank, self.world = rank, world

    def shard_finalize(self):
        self._check(self._L.lutamm_shard_finalize(self._h))

    def amm_column_sharded(self, layer_id: int, input_tensor, gathered, n_tokens: int | None = None,
                           search_mode: int = SHARD_SEARCH_REPLICATED, flags: int = 0):
        """This rank's column slab of the AMM into block `rank` of gathered [G][n_tokens][N/G], then one in-place
        all-gather (the lut_parallelism axis of the reference, pim_lut_host.cpp:26-37)."""
        M = int(n_tokens if n_tokens is not None else input_tensor.shape[0])
        self._check(self._L.lutamm_amm_column_sharded(self._h, layer_id, _ptr(input_tensor), _ptr(gathered), M, search_mode, flags))

    def shard_alloc_gathered(self, world: int, n_tokens: int, n_local: int):
        """A gathered-output buffer [world][n_tokens][n_local] fp32 that every rank can store into (collective call;
        CUDA IPC).  Returns a torch tensor view of it; release with shard_free_gathered(tensor)."""
        import torch
        nbytes = 4 * world * n_tokens * n_local
        ptr = ctypes.c_void_p()
        self._check(self._L.lutamm_shard_alloc_gathered(self._h, nbytes, ctypes.byref(ptr)))

        class _Mem:   # the CUDA array interface lets torch wrap memory it did not allocate
            __cuda_array_interface__ = {"shape": (world, n_tokens, n_local), "typestr": "<f4", "data": (ptr.value, False), "version": 3,
                                        "strides": None}
        holder = _Mem()
        t = torch.as_tensor(holder, device=torch.device("cuda", self.device))
        t._lutamm_base = ptr.value
        return t

    def shard_free_gathered(self, tensor):
        self._check(self._L.lutamm_shard_free_gathered(self._h, ctypes.c_void_p(tensor._lutamm_base)))

    def amm_token_sharded(self, layer_id: int, input_rows, output, n_tokens_total: int, gather: bool = False, flags: int = 0):
        """This rank's tokens of the AMM (the input_parallelism axis, pim_lut_host.cpp:109-117); with gather=True
        `output` is the full [n_tokens_total][N] on every rank."""
        self._check(self._L.lutamm_amm_token_sharded(self._h, layer_id, _ptr(input_rows), _ptr(output), n_tokens_total,
                                                     1 if gather else 0, flags))

    def tune_sharding(self, layer_all_columns: int, layer_my_columns: int, n_tokens_total: int, reps: int = 3) -> dict:
        """Times the shardings of one operator on this group of GPUs (a collective call; the auto-tuner's choice of
        input_parallelism x lut_parallelism, auto_tuner.cpp:368-549, by measurement).  Pass -1 for a layer that is not
        loaded.  Returns {"best": name, "world": G, "ms": {name: ms per call of the slowest rank, or None}}."""
        r = ShardingReport()
        self._check(self._L.lutamm_tune_sharding(self._h, layer_all_columns, layer_my_columns, n_tokens_total, reps, ctypes.byref(r)))
        return {"best": SHARDING_MODES[r.best], "world": int(r.world),
                "ms": {n: (float(r.ms[i]) if r.ms[i] >= 0 else None) for i, n in enumerate(SHARDING_MODES)}}

    # -- plans / tuning / timing
    def set_plan(self, layer_id: int, **kw):
        p = Plan()
        for k, v in kw.items():
            setattr(p, k, v)
        self._check(self._L.lutamm_set_plan(self._h, layer_id, ctypes.byref(p)))

    def set_activation(self, layer_id: int, activation: int):
        """Activation fused into the LUT kernel's epilogue: ACT_NONE, ACT_GELU_TANH or ACT_GELU_TANH_F16."""
        self._check(self._L.lutamm_set_activation(self._h, layer_id, activation))

    def get_plan(self, layer_id: int) -> dict:
        p = Plan()
        self._check(self._L.lutamm_get_plan(self._h, layer_id, ctypes.byref(p)))
        return p.as_dict()

    def tune(self, layer_id: int, n_tokens: int) -> dict:
        p = Plan()
        self._check(self._L.lutamm_tune(self._h, layer_id, n_tokens, ctypes.byref(p)))
        return p.as_dict()

    def measure_int8_peak(self) -> dict:
        """The GPU's int8 tensor rate, measured by a few milliseconds of nothing but tcgen05.mma kind::i8."""
        tops, mac, mhz = ctypes.c_double(), ctypes.c_double(), ctypes.c_double()
        self._check(self._L.lutamm_measure_int8_peak(self._h, ctypes.byref(tops), ctypes.byref(mac), ctypes.byref(mhz)))
        return {"tops": tops.value, "mac_per_clk_sm": mac.value, "sm_mhz": mhz.value}

    def plan_cache_save(self, path: str):
        """Write the plans lutamm_tune has found in this context, keyed by shape and SM count, to a text file."""
        self._check(self._L.lutamm_plan_cache_save(self._h, path.encode()))

    def plan_cache_load(self, path: str):
        self._check(self._L.lutamm_plan_cache_load(self._h, path.encode()))

    def enable_timing(self, on: bool = True):
        self._check(self._L.lutamm_enable_timing(self._h, 1 if on else 0))

    def timings(self) -> dict:
        t = Timings()
        self._check(self._L.lutamm_get_timings(self._h, ctypes.byref(t)))
        return {k: getattr(t, k) for k, _ in Timings._fields_}
