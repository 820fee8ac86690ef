"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache, one
function for each part, NumPy only. It shares no code with the library; the tests compare the
library with it.

It rests on the formulas of the reference's scalar CPU backend and decoder (each function
cites the file and lines, paths as in the reference project), with that backend's rounding
points: sums in float64, results stored as float32. The reference's model code is Pascal and
cannot be compiled or imported here; ``tests/golden/`` holds the record of this file checked
once against the reference's checked-in ``tiny-qwen3`` fixtures (transformers FP32 logits).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np

f32 = np.float32
f64 = np.float64


# ----------------------------------------------------------------------------- files
def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """Every tensor of a safetensors file as float32 (BF16 widened exactly: a BF16 value is the
    upper half of a float32, src/infer/mormot.ai.infer.tensor.pas:483)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, e_ = e["data_offsets"]
        raw = data[b:e_]
        if e["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            a = u.view(np.float32)
        elif e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype=np.float32)
        else:
            raise ValueError(f"{name}: {e['dtype']}")
        out[name] = a.reshape(e["shape"]).copy()
    return out


def read_model_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    return config, read_safetensors(os.path.join(folder, "model.safetensors"))


# ----------------------------------------------------------------------------- parts
def embed(table: np.ndarray, ids: Sequence[int]) -> np.ndarray:
    """x[i,:] = E[id_i,:], no scaling (src/infer/mormot.ai.infer.decoder.pas:3292-3309)."""
    ids = np.asarray(ids, dtype=np.int64)
    if ids.size == 0 or ids.min() < 0 or ids.max() >= table.shape[0]:
        raise ValueError("token id out of range")
    return table[ids].astype(f32)


def inverse_frequencies(theta: float, rot_dim: int) -> np.ndarray:
    """inv_freq[i] = 1 / f32(theta ^ f32(2i/d)), stored as float32
    (src/infer/mormot.ai.infer.decoder.pas:1733-1736)."""
    out = np.empty(rot_dim // 2, dtype=f32)
    for i in range(rot_dim // 2):
        e = f32((2 * i) / rot_dim)
        out[i] = f32(1.0 / f64(f32(math.exp(math.log(theta) * f64(e)))))
    return out


def rotary_tables(inv_freq: np.ndarray, positions: Sequence[int]):
    """angle = f32(inv_freq[i] * pos); cos, sin rounded to float32
    (src/infer/mormot.ai.infer.decoder.pas:2539-2561)."""
    pos = np.asarray(positions, dtype=f32)[:, None]
    angle = (inv_freq[None, :] * pos).astype(f32)
    return np.cos(angle.astype(f64)).astype(f32), np.sin(angle.astype(f64)).astype(f32)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """inv = 1/sqrt(sum(x^2)/cols + eps) in float64; n = f32(x*inv); y = f32(w*n)
    (src/infer/mormot.ai.infer.backend.cpu.pas:1769-1795)."""
    xd = x.astype(f64)
    inv = 1.0 / np.sqrt((xd * xd).sum(axis=-1, keepdims=True) / x.shape[-1] + eps)
    n = (xd * inv).astype(f32)
    return (w.astype(f32) * n).astype(f32)


def linear(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """y = x · Wᵀ for a weight [out, in], float64 accumulation, no bias
    (src/infer/mormot.ai.infer.backend.cpu.pas:1548-1565)."""
    return (x.astype(f64) @ w.astype(f64).T).astype(f32)


def rope(x: np.ndarray, heads: int, head_dim: int, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """rotate_half over the whole head: x'[i] = x[i]c - x[i+h]s; x'[i+h] = x[i+h]c + x[i]s
    (src/infer/mormot.ai.infer.backend.cpu.pas:1862-1888)."""
    n = x.shape[0]
    half = cos.shape[1]
    v = x.reshape(n, heads, head_dim).astype(f64)
    a = v[:, :, :half].copy()
    b = v[:, :, half:2 * half].copy()
    c = cos.astype(f64)[:, None, :]
    s = sin.astype(f64)[:, None, :]
    v[:, :, :half] = a * c - b * s
    v[:, :, half:2 * half] = b * c + a * s
    return v.astype(f32).reshape(n, heads * head_dim)


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, heads: int, kv_heads: int,
                     head_dim: int, window: int = 0, scale: Optional[float] = None) -> np.ndarray:
    """Causal grouped-query attention of a whole sequence (past 0): head h reads KV head
    h div (heads div kv_heads); keys max(0, r+1-window)..r; s = q·k·scale, p = exp(s-max),
    y = (sum p v)/(sum p), all in float64, stored as float32
    (src/infer/mormot.ai.infer.backend.cpu.pas:1296-1353, :1377-1380)."""
    n = q.shape[0]
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    qh = q.reshape(n, heads, head_dim).astype(f64)
    kh = k.reshape(n, kv_heads, head_dim).astype(f64)
    vh = v.reshape(n, kv_heads, head_dim).astype(f64)
    y = np.zeros((n, heads, head_dim), dtype=f32)
    rep = heads // kv_heads
    for h in range(heads):
        g = h // rep
        for r in range(n):
            total = r + 1
            first = total - window if (window > 0 and total > window) else 0
            s = (kh[first:total, g, :] @ qh[r, h, :]) * scale
            p = np.exp(s - s.max())
            y[r, h, :] = ((p @ vh[first:total, g, :]) * (1.0 / p.sum())).astype(f32)
    return y.reshape(n, heads * head_dim)


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """a = f32(g / (1 + exp(-g))) · u (src/infer/mormot.ai.infer.backend.cpu.pas:1827-1833)."""
    g = gate.astype(f64)
    b = (g / (1.0 + np.exp(-g))).astype(f32)
    return (b * up.astype(f32)).astype(f32)


# ----------------------------------------------------------------------------- blocks
def layer_windows(config: dict) -> List[int]:
    """The window of each layer (src/infer/mormot.ai.infer.model.qwen3.pas:327-403)."""
    layers = config["num_hidden_layers"]
    w = 0
    if config.get("use_sliding_window"):
        w = 4096 if "sliding_window" not in config else (config["sliding_window"] or 0)
    out = [0] * layers
    types = config.get("layer_types")
    if isinstance(types, list):
        return [w if t == "sliding_attention" else 0 for t in types]
    if w:
        for i in range(max(config.get("max_window_layers", 28), 0), layers):
            out[i] = w
    return out


def rope_theta(config: dict) -> float:
    rp = config.get("rope_parameters")
    return float(rp["rope_theta"] if isinstance(rp, dict) else config["rope_theta"])


def attention_block(x, w, p, config, cos, sin, window, states=None):
    """H = norm(X); Q,K,V = H·Wᵀ; per-head q_norm/k_norm; RoPE on Q and K; attention;
    X += Attn·Woᵀ (src/infer/mormot.ai.infer.decoder.pas:2625-2702)."""
    nh, nkv, hd = (config["num_attention_heads"], config["num_key_value_heads"],
                   config["head_dim"])
    eps = config["rms_norm_eps"]
    n = x.shape[0]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = linear(h, w[p + "self_attn.q_proj.weight"])
    k = linear(h, w[p + "self_attn.k_proj.weight"])
    v = linear(h, w[p + "self_attn.v_proj.weight"])
    q = rms_norm(q.reshape(n * nh, hd), w[p + "self_attn.q_norm.weight"], eps).reshape(n, nh * hd)
    k = rms_norm(k.reshape(n * nkv, hd), w[p + "self_attn.k_norm.weight"], eps).reshape(n, nkv * hd)
    q = rope(q, nh, hd, cos, sin)
    k = rope(k, nkv, hd, cos, sin)
    a = causal_attention(q, k, v, nh, nkv, hd, window)
    t = linear(a, w[p + "self_attn.o_proj.weight"])
    if states is not None:
        states["attn"] = t
        states["q"], states["k"], states["v"], states["a"] = q, k, v, a
    return (x + t).astype(f32)


def dense_block(x, w, p, config, states=None):
    """H = norm(X); X += (silu(H·Wgᵀ)·(H·Wuᵀ))·Wdᵀ
    (src/infer/mormot.ai.infer.decoder.pas:2865-2899)."""
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], config["rms_norm_eps"])
    g = linear(h, w[p + "mlp.gate_proj.weight"])
    u = linear(h, w[p + "mlp.up_proj.weight"])
    t = linear(swiglu(g, u), w[p + "mlp.down_proj.weight"])
    if states is not None:
        states["mlp"] = t
    return (x + t).astype(f32)


def forward(config: dict, w: Dict[str, np.ndarray], ids: Sequence[int],
            states: Optional[dict] = None) -> np.ndarray:
    """Logits [n, vocab] of one whole sequence from position 0
    (src/infer/mormot.ai.infer.decoder.pas:3245-3369). ``states`` receives the intermediate
    states under the names of the reference's fixtures (embed, layerNN, layer00_attn, ...)."""
    hd = config["head_dim"]
    inv = inverse_frequencies(rope_theta(config), hd)
    cos, sin = rotary_tables(inv, range(len(ids)))
    x = embed(w["model.embed_tokens.weight"], ids)
    if states is not None:
        states["embed"] = x
    for l, window in enumerate(layer_windows(config)):
        p = f"model.layers.{l}."
        st = {} if states is not None else None
        x = attention_block(x, w, p, config, cos, sin, window, st)
        x = dense_block(x, w, p, config, st)
        if states is not None:
            states[f"layer{l:02d}_attn"] = st["attn"]
            states[f"layer{l:02d}_mlp"] = st["mlp"]
            states[f"layer{l:02d}"] = x
    hN = rms_norm(x, w["model.norm.weight"], config["rms_norm_eps"])
    if states is not None:
        states["norm"] = hN
    head = (w["model.embed_tokens.weight"] if config.get("tie_word_embeddings")
            else w["lm_head.weight"])
    return linear(hN, head)


# ----------------------------------------------------------------------------- sampling
def arg_max(values: np.ndarray) -> int:
    """The highest value, the lowest index on ties, a NaN never chosen unless all are NaN;
    -0 equals +0 (src/infer/mormot.ai.infer.sampler.pas:123-159)."""
    best = -1
    for i, v in enumerate(values):
        if math.isnan(v):
            continue
        if best < 0 or v > values[best]:
            best = i
    return max(best, 0)


class PlainSampler:
    """Temperature, top-k, top-p, min-p, then one draw from a splitmix64 stream
    (src/infer/mormot.ai.infer.sampler.pas:222-233 for the generator, :280-436 for Next)."""

    def __init__(self, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, seed=0):
        bad = (any(math.isnan(v) or math.isinf(v) for v in (temperature, top_p, min_p))
               or top_k < 0 or top_p <= 0 or top_p > 1 or min_p < 0 or min_p >= 1)
        if bad:
            raise ValueError("sampling settings")
        self.temperature, self.top_k, self.top_p, self.min_p = temperature, top_k, top_p, min_p
        self.state = seed & 0xFFFFFFFFFFFFFFFF

    def next_double(self) -> float:
        m = 0xFFFFFFFFFFFFFFFF
        self.state = (self.state + 0x9E3779B97F4A7C15) & m
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        z = z ^ (z >> 31)
        return (z >> 11) * (1.0 / 9007199254740992.0)

    def next(self, logits: np.ndarray) -> int:
        if self.temperature <= 0:
            return arg_max(logits)
        best = arg_max(logits)
        m = float(logits[best])
        if math.isnan(m) or math.isinf(m) or self.temperature < 1e-30:
            return best
        lg = logits.astype(f64)
        finite = np.isfinite(lg)
        probs = np.where(finite, np.exp((np.where(finite, lg, m) - m) / self.temperature), 0.0)
        probs = probs / probs.sum()
        if self.top_k == 0 and self.top_p >= 1 and self.min_p == 0:
            u = self.next_double()
            cum = 0.0
            for i, p in enumerate(probs):
                cum += p
                if p > 0 and u < cum:
                    return i
            return best
        # candidates in the order: higher logit first, lower id on a tie
        cand = [i for i in range(len(lg)) if finite[i]]
        cand.sort(key=lambda i: (-lg[i], i))
        n = len(cand)
        if self.top_k > 0 and n > self.top_k:
            keep = self.top_k
            while keep < n and lg[cand[keep]] == lg[cand[self.top_k - 1]]:
                keep += 1
            n = keep
        if self.top_p < 1:
            mass = sum(probs[cand[i]] for i in range(n)) if self.top_k > 0 else 1.0
            cum, keep = 0.0, n
            for i in range(n):
                cum += probs[cand[i]]
                if cum >= self.top_p * mass:
                    keep = i + 1
                    break
            n = keep
        if self.min_p > 0:
            keep = 1
            while keep < n and probs[cand[keep]] >= self.min_p * probs[cand[0]]:
                keep += 1
            n = keep
        total = sum(probs[cand[i]] for i in range(n))
        u = self.next_double() * total
        cum = 0.0
        for i in range(n):
            cum += probs[cand[i]]
            if u < cum:
                return cand[i]
        return cand[0]


def greedy(config: dict, w: Dict[str, np.ndarray], prompt: Sequence[int], max_new: int,
           stop: Sequence[int] = ()) -> List[int]:
    """Greedy generation by whole-sequence passes; the stop token is returned
    (src/infer/mormot.ai.infer.decoder.pas:3390-3426)."""
    ids = list(prompt)
    out: List[int] = []
    while len(out) < max_new:
        nxt = arg_max(forward(config, w, ids)[-1])
        out.append(nxt)
        if nxt in stop or len(ids) >= config["max_position_embeddings"]:
            break
        ids.append(nxt)
    return out
