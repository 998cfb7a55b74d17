"""Seeded synthetic tensors for the LUT-AMM benchmark and parity cases.

The reference measures on random tensors too (inference-engine/test/test_amm.cpp:26-67),
but from one std::mt19937 shared by racing OpenMP threads, so its data cannot be
reproduced.  Here every tensor has its own generator spawned from one SeedSequence:
activations fp32 N(0,1), centroids fp32 N(0,1) [CB][CT][v], LUT int8 uniform in
[-127,127] [CB][CT][N], bias fp32 N(0,0.02) [N]; scale 0.01 and LUT bias 0 by default.
`reference_style=True` gives the reference driver's own ranges instead
(U(-5,5) / U(-10,10) / int8 U[-128,127], test_amm.cpp:30,40,50-53,63).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class AmmCase:
    x: np.ndarray          # [M][K] fp32
    centroid: np.ndarray   # [CB][CT][v] fp32
    lut: np.ndarray        # [CB][CT][N] int8
    bias: np.ndarray       # [N] fp32
    scale: float
    lut_bias: float

    @property
    def M(self): return self.x.shape[0]
    @property
    def K(self): return self.x.shape[1]
    @property
    def CB(self): return self.centroid.shape[0]
    @property
    def CT(self): return self.centroid.shape[1]
    @property
    def v(self): return self.centroid.shape[2]
    @property
    def N(self): return self.lut.shape[2]


def make_weights(K: int, N: int, v: int, CT: int, seed=0, stream: int = 0, reference_style: bool = False):
    """(centroid, lut, bias) for one linear layer; `stream` separates layers under one seed."""
    assert K % v == 0
    CB = K // v
    ss = np.random.SeedSequence([seed, 1000 + stream]) if stream else np.random.SeedSequence(seed)
    _, s_c, s_l, s_b = ss.spawn(4)
    if reference_style:
        centroid = np.random.default_rng(s_c).uniform(-10, 10, (CB, CT, v)).astype(np.float32)
        lut = np.random.default_rng(s_l).integers(-128, 128, (CB, CT, N), dtype=np.int8)
        bias = np.random.default_rng(s_b).uniform(-10, 10, (N,)).astype(np.float32)
    else:
        centroid = np.random.default_rng(s_c).standard_normal((CB, CT, v), dtype=np.float32)
        lut = np.random.default_rng(s_l).integers(-127, 128, (CB, CT, N), dtype=np.int8)
        bias = (np.random.default_rng(s_b).standard_normal((N,), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    return centroid, lut, bias


def make_input(M: int, K: int, seed=0, stream: int = 0, reference_style: bool = False) -> np.ndarray:
    ss = np.random.SeedSequence([seed, 1000 + stream]) if stream else np.random.SeedSequence(seed)
    s_x = ss.spawn(4)[0]
    rng = np.random.default_rng(s_x)
    if reference_style:
        return rng.uniform(-5, 5, (M, K)).astype(np.float32)
    return rng.standard_normal((M, K), dtype=np.float32)


def make_case(M: int, K: int, N: int, v: int, CT: int, seed=0, scale: float = 0.01, lut_bias: float = 0.0,
              reference_style: bool = False, stream: int = 0) -> AmmCase:
    centroid, lut, bias = make_weights(K, N, v, CT, seed, stream, reference_style)
    x = make_input(M, K, seed, stream, reference_style)
    return AmmCase(x, centroid, lut, bias, float(np.float32(scale)), float(np.float32(lut_bias)))


# benchmark workloads ---------------------------------------------------------------------
# name -> (M, [(linear name, K, N)], v, CT)
BERT_BASE = [("qkv", 768, 2304), ("o", 768, 768), ("ffn1", 768, 3072), ("ffn2", 3072, 768)]
BERT_LARGE = [("qkv", 1024, 3072), ("o", 1024, 1024), ("ffn1", 1024, 4096), ("ffn2", 4096, 1024)]

WORKLOADS = {
    "c1": dict(M=512, linears=[("ffn1", 768, 3072)], v=2, CT=16,
               what="single LUT-AMM linear, BERT-base FFN1 shape, M=512"),
    "c2": dict(M=1024, linears=BERT_BASE, v=2, CT=16,
               what="the four LUT-AMM linears of one BERT-base encoder layer, batch 8 x seq 128"),
    "c3": dict(M=8192, linears=BERT_LARGE, v=4, CT=16,
               what="the four LUT-AMM linears of one BERT-large encoder layer, batch 16 x seq 512"),
    "c4": dict(M=12608, linears=BERT_BASE, v=2, CT=16,
               what="the four LUT-AMM linears of one ViT-Base/16 layer, batch 64 x 197 tokens"),
    "c5": dict(M=65536, linears=[("amm", 4096, 16384)], v=2, CT=16,
               what="large-M AMM, M=65536 K=4096 N=16384"),
}


def algorithmic_bytes(M: int, K: int, N: int, v: int, CT: int) -> dict:
    """Compulsory HBM traffic of one AMM with uint8 indices."""
    CB = K // v
    a = 4 * M * K + 4 * CB * CT * v + M * CB
    b = M * CB + CB * CT * N + 4 * N + 4 * M * N
    return {"ccs": a, "lut": b, "total": a + b}
