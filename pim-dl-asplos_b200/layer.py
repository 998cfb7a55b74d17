"""Encoder layer and model built on the LUT-AMM operator: the callers of the hot path.

Mirrors pim_lut_transformer_layer() (inference-engine/src/host/transformer_layer.cpp:263-625)
and transformer_inference() (transformer_model.cpp:13-49) of the reference:

    qkv   = AMM_qkv(x)                       [n, 3*token_dim], columns ordered Q | K | V
            (or, in the reference's SEPARATE build - the one its model driver uses, run_model.py:130 -
             q = AMM_q(x), k = AMM_k(x), v = AMM_v(x): three operators of their own, :333-343)
    att   = softmax(Q K^T / sqrt(head_dim)) V   per (batch, head), no mask (:217-229)
    o     = AMM_o(att)
    h     = x + LayerNorm_1(o)               eps 1e-6 (:50-90); note: norm of the projection,
    f     = GELU(AMM_ffn1(h))                    then the residual - not LayerNorm(x + o)
    y     = h + LayerNorm_2(AMM_ffn2(f))

The four linears run in the CUDA library through the C ABI; attention, LayerNorm and the
residual adds are plain PyTorch on the same stream (they stay dense fp32, as in the
reference, where they run in ggml on the host).  The GELU after FFN1 - a separate in-place
pass in the reference (:503) - is applied inside the FFN1 operator's epilogue
(`fused_gelu`, lutamm_set_activation), which saves one read and one write of [n, ffn_dim].  All the loops of the reference that move
data between the DPU-tiled layout and row-major (:97-208, :449-471, :520-542, :574-596)
have no counterpart: every tensor here is row-major.

The reference's GELU is ggml's (a tanh approximation evaluated through an fp16 table); ggml
is not part of the reference tree, so the layer's output is not pinned bit for bit - the AMM
results inside it are.
"""
from __future__ import annotations

import numpy as np

from . import ACT_GELU_TANH, FLAG_ASYNC, LutAmmContext, synth

LINEARS = ("qkv", "o", "ffn1", "ffn2")
SEPARATE_LINEARS = ("q", "k", "v", "o", "ffn1", "ffn2")

# .npz keys written by model-calibration/pim_weight_converter.py:86-96 and read by
# test/test_transformer.cpp:252-462, per layer index L.  A converted HuggingFace checkpoint has the three
# projections query / key / value (the reference's SEPARATE build reads those, test_transformer.cpp:295-368);
# a file with one fused "qkv" operator is what its non-SEPARATE build reads (:259-286).
NPZ_PREFIX = {
    "qkv": "{L}.attention.self.qkv",
    "q": "{L}.attention.self.query",
    "k": "{L}.attention.self.key",
    "v": "{L}.attention.self.value",
    "o": "{L}.attention.output.dense",
    "ffn1": "{L}.intermediate.dense",
    "ffn2": "{L}.output.dense",
}
NPZ_NORM = {"ln1": "{L}.attention.output.LayerNorm", "ln2": "{L}.output.LayerNorm"}


def linear_shapes(token_dim: int, ffn_hidden_dim: int):
    return {"qkv": (token_dim, 3 * token_dim), "o": (token_dim, token_dim),
            "q": (token_dim, token_dim), "k": (token_dim, token_dim), "v": (token_dim, token_dim),
            "ffn1": (token_dim, ffn_hidden_dim), "ffn2": (ffn_hidden_dim, token_dim)}


def _per_linear(d: dict, name: str):
    """Codebook / centroid counts of a linear; Q, K and V take the attention-output operator's, as the
    reference's parser fills them (src/host/parser.cpp:235-322)."""
    return d[name] if name in d else d["o"]


def random_layer_weights(token_dim, ffn_hidden_dim, num_codebook: dict, num_centroid: dict, seed=0, layer=0,
                         scale=0.01, lut_bias=0.0, separate_qkv: bool = False):
    """Synthetic weights for one layer: {name: (centroid, lut, bias, scale, lut_bias)} + LayerNorm."""
    w = {}
    for li, name in enumerate(SEPARATE_LINEARS if separate_qkv else LINEARS):
        K, N = linear_shapes(token_dim, ffn_hidden_dim)[name]
        CB, CT = _per_linear(num_codebook, name), _per_linear(num_centroid, name)
        cen, lut, bias = synth.make_weights(K, N, K // CB, CT, seed=seed, stream=1 + layer * 8 + li)
        w[name] = (cen, lut, bias, scale, lut_bias)
    w["ln1"] = (np.ones(token_dim, np.float32), np.zeros(token_dim, np.float32))
    w["ln2"] = (np.ones(token_dim, np.float32), np.zeros(token_dim, np.float32))
    return w


def load_layer_weights_npz(npz, layer: int, token_dim, ffn_hidden_dim, num_codebook: dict, num_centroid: dict,
                           separate_qkv: bool | None = None):
    """One layer from a converted checkpoint (keys as in test_transformer.cpp:252-462).  The LUT is
    stored [CB*CT][N] (pim_weight_converter.py:90) - the canonical [CB][CT][N] flattened.

    separate_qkv: None = by what the file holds (a fused "qkv" operator if present, else the three
    projections); True / False = require that form.  Three projections can only be merged into one QKV
    operator when they share one set of centroids and one quantisation scale, which a calibrated
    checkpoint does not; such a file is run as three operators, like the reference's SEPARATE build."""
    files = set(npz.files) if hasattr(npz, "files") else set(npz.keys())
    have_fused = NPZ_PREFIX["qkv"].format(L=layer) + ".lut.tensor" in files
    have_sep = NPZ_PREFIX["q"].format(L=layer) + ".lut.tensor" in files
    if separate_qkv is None:
        separate_qkv = not have_fused
    if separate_qkv and not have_sep:
        raise KeyError(f"layer {layer}: no attention.self.query/key/value operators in the checkpoint")
    if not separate_qkv and not have_fused:
        raise KeyError(f"layer {layer}: no fused attention.self.qkv operator in the checkpoint (it holds query/key/value: "
                       "load with separate_qkv=True)")
    w = {}
    for name in (SEPARATE_LINEARS if separate_qkv else LINEARS):
        K, N = linear_shapes(token_dim, ffn_hidden_dim)[name]
        CB, CT = _per_linear(num_codebook, name), _per_linear(num_centroid, name)
        p = NPZ_PREFIX[name].format(L=layer)
        cen = np.ascontiguousarray(npz[p + ".centroids.weight"], dtype=np.float32)
        if cen.size != CB * CT * (K // CB):
            raise ValueError(f"{p}: {cen.size} centroid values, expected num_codebook {CB} x num_centroid {CT} x {K // CB}")
        cen = cen.reshape(CB, CT, K // CB)
        lut = np.ascontiguousarray(npz[p + ".lut.tensor"]).astype(np.int8).reshape(CB, CT, N)
        bias = np.ascontiguousarray(npz[p + ".bias"], dtype=np.float32).reshape(N)
        w[name] = (cen, lut, bias, float(np.asarray(npz[p + ".lut.scale"]).reshape(-1)[0]),
                   float(np.asarray(npz[p + ".lut.bias"]).reshape(-1)[0]))
    for k, p in NPZ_NORM.items():
        p = p.format(L=layer)
        w[k] = (np.ascontiguousarray(npz[p + ".weight"], dtype=np.float32), np.ascontiguousarray(npz[p + ".bias"], dtype=np.float32))
    return w


def checkpoint_layer_count(npz) -> int:
    files = npz.files if hasattr(npz, "files") else npz.keys()
    ids = {int(k.split(".")[0]) for k in files if k.split(".")[0].isdigit()}
    return max(ids) + 1 if ids else 0


class LutTransformerLayer:
    """One encoder layer; `forward` takes and returns a device tensor [n, token_dim]."""

    def __init__(self, ctx: LutAmmContext, weights: dict, seq_len: int, batch_size: int, head_num: int,
                 first_layer_id: int = 0, plans: dict | None = None, fused_gelu: bool = True):
        import torch
        self.ctx, self.torch = ctx, torch
        self.seq_len, self.batch, self.heads = seq_len, batch_size, head_num
        self.n = seq_len * batch_size
        self.ids = {}
        self.separate_qkv = "qkv" not in weights
        self.linears = SEPARATE_LINEARS if self.separate_qkv else LINEARS
        for k, name in enumerate(self.linears):
            cen, lut, bias, scale, lut_bias = weights[name]
            lid = first_layer_id + k
            ctx.load_weights(lid, cen, lut, bias, scale, lut_bias)
            plan = (plans or {}).get(name) or ((plans or {}).get("o") if name in ("q", "k", "v") else None)
            if plan:
                ctx.set_plan(lid, **plan)
            self.ids[name] = lid
        self.fused_gelu = fused_gelu
        if fused_gelu:
            ctx.set_activation(self.ids["ffn1"], ACT_GELU_TANH)
        self.token_dim = weights["o"][1].shape[2]
        self.ffn_dim = weights["ffn1"][1].shape[2]
        dev = torch.device("cuda", ctx.device)
        self.ln = {k: tuple(torch.from_numpy(a).to(dev) for a in weights[k]) for k in ("ln1", "ln2")}
        f32 = dict(device=dev, dtype=torch.float32)
        self.buf = {"o": torch.empty(self.n, self.token_dim, **f32),
                    "ffn1": torch.empty(self.n, self.ffn_dim, **f32), "ffn2": torch.empty(self.n, self.token_dim, **f32)}
        if self.separate_qkv:
            for name in ("q", "k", "v"):
                self.buf[name] = torch.empty(self.n, self.token_dim, **f32)
        else:
            self.buf["qkv"] = torch.empty(self.n, 3 * self.token_dim, **f32)
        self.amm_ms = 0.0

    def tune(self):
        return {name: self.ctx.tune(self.ids[name], self.n) for name in self.linears}

    def _amm(self, name, x):
        self.ctx.amm_host(self.ids[name], x, self.buf[name], n_tokens=self.n, flags=FLAG_ASYNC)
        return self.buf[name]

    def forward(self, x):
        """x: contiguous fp32 [n, token_dim] on the context's device; runs on torch's current
        stream, which must be the stream given to ctx.set_stream()."""
        torch, F = self.torch, self.torch.nn.functional
        B, S, H, D = self.batch, self.seq_len, self.heads, self.token_dim
        hd = D // H
        if self.separate_qkv:   # three operators on the same input (transformer_layer.cpp:333-343)
            q, k, v = (self._amm(name, x).reshape(B, S, H, hd).transpose(1, 2) for name in ("q", "k", "v"))
        else:
            qkv = self._amm("qkv", x)
            q, k, v = (t.reshape(B, S, H, hd).transpose(1, 2) for t in qkv.split(D, dim=1))
        att = F.scaled_dot_product_attention(q, k, v)                    # 1/sqrt(head_dim), no mask
        att = att.transpose(1, 2).reshape(self.n, D).contiguous()
        o = self._amm("o", att)
        h = x + F.layer_norm(o, (D,), self.ln["ln1"][0], self.ln["ln1"][1], eps=1e-6)
        f = self._amm("ffn1", h.contiguous())
        if not self.fused_gelu:
            f = F.gelu(f, approximate="tanh")
        y = h + F.layer_norm(self._amm("ffn2", f), (D,), self.ln["ln2"][0], self.ln["ln2"][1], eps=1e-6)
        return y


class LutTransformer:
    """layer_num encoder layers back to back (transformer_model.cpp:13-49)."""

    def __init__(self, ctx, layer_weights: list, seq_len, batch_size, head_num, plans=None, fused_gelu=True):
        self.layers = [LutTransformerLayer(ctx, w, seq_len, batch_size, head_num, first_layer_id=8 * i, plans=plans,
                                           fused_gelu=fused_gelu)
                       for i, w in enumerate(layer_weights)]

    def forward(self, x):
        for layer in self.layers:
            x = layer.forward(x)
        return x


def reference_layer_numpy(x, weights, seq_len, batch_size, head_num, amm):
    """The same dataflow in numpy/float64-free fp32, for tests: `amm(name, x)` supplies the four
    linears (the CPU oracle in the test-suite).  Not used by the library."""
    n, D = x.shape
    hd = D // head_num

    def ln(t, wb):
        mean = t.astype(np.float64).sum(1, keepdims=True) / D
        c = (t - mean.astype(np.float32)).astype(np.float32)
        var = (c.astype(np.float64) ** 2).sum(1, keepdims=True) / D
        return (c * (1.0 / np.sqrt(var.astype(np.float32) + np.float32(1e-6))).astype(np.float32) * wb[0] + wb[1]).astype(np.float32)

    if "qkv" in weights:
        qkv3 = np.split(amm("qkv", x), 3, axis=1)
    else:
        qkv3 = [amm(name, x) for name in ("q", "k", "v")]
    q, k, v = (t.reshape(batch_size, seq_len, head_num, hd).transpose(0, 2, 1, 3) for t in qkv3)
    s = (q @ k.transpose(0, 1, 3, 2)) / np.float32(np.sqrt(hd))
    s = np.exp(s - s.max(-1, keepdims=True))
    p = (s / s.sum(-1, keepdims=True)).astype(np.float32)
    att = (p @ v).transpose(0, 2, 1, 3).reshape(n, D).astype(np.float32)
    o = amm("o", np.ascontiguousarray(att))
    h = (x + ln(o, weights["ln1"])).astype(np.float32)
    f1 = amm("ffn1", np.ascontiguousarray(h))
    g = (0.5 * f1 * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (f1 + 0.044715 * f1 ** 3)))).astype(np.float32)
    y = (h + ln(amm("ffn2", np.ascontiguousarray(g)), weights["ln2"])).astype(np.float32)
    return y
