"""Plain, slow implementation of the Bigerax decoder in numpy float64: whole sequences, no cache, one function per
mechanism.  It is the oracle of the Bigerax tests and shares no code with the package.

Notation: ``T`` tokens, width ``D``; a linear map stored ``[out, in]`` is applied as ``x @ W.T (+ b)``.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional

import numpy as np


# ---- container --------------------------------------------------------------------------------------------------
def _bf16_to_f64(raw: bytes, shape) -> np.ndarray:
    u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
    return u16.view(np.float32).astype(np.float64).reshape(shape)


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw, shape = data[lo:hi], tuple(info["shape"])
        dt = info["dtype"]
        if dt == "BF16":
            out[name] = _bf16_to_f64(raw, shape)
        elif dt == "F32":
            out[name] = np.frombuffer(raw, dtype="<f4").astype(np.float64).reshape(shape)
        elif dt == "I32":
            out[name] = np.frombuffer(raw, dtype="<i4").astype(np.int64).reshape(shape)
        else:
            raise ValueError(f"dtype {dt} of '{name}' is not read by the oracle")
    return out


def load_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# ---- mechanisms ---------------------------------------------------------------------------------------------------
def bigram_embedding(tokens, embed, bigram, buckets: int, mul_prev: int, mul_cur: int, prev: Optional[int] = None):
    """Token row plus a hashed row for the pair (previous token, token); the pair of a sequence's first token (no
    ``prev``) is the extra last row of the table."""
    x = np.zeros((len(tokens), embed.shape[1]))
    for t, tok in enumerate(tokens):
        p = prev if t == 0 else tokens[t - 1]
        row = buckets if p is None else (int(p) * mul_prev + int(tok) * mul_cur) % buckets
        x[t] = embed[tok] + bigram[row]
    return x


def group_rmsnorm(x, w, groups: int, eps: float):
    """Every one of ``groups`` equal consecutive parts of a row is divided by its own root mean square."""
    T, D = x.shape
    parts = x.reshape(T, groups, D // groups)
    parts = parts / np.sqrt((parts * parts).mean(axis=-1, keepdims=True) + eps)
    return parts.reshape(T, D) * w


def rotate_pairs(x, positions, dims: int, base: float):
    """x [T, heads, size]: dimensions 2i and 2i+1 (i < dims/2) turn by the angle position * base^(-2i/dims)."""
    out = x.copy()
    i = np.arange(dims // 2)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * base ** (-2.0 * i / dims)     # [T, dims/2]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def window_sink_attention(q, k, v, scale: float, window: int):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of one whole sequence.  Query i sees keys j with 0 <= i - j < window
    (window 0: all earlier ones); the weights are exp(s) / (1 + sum exp(s)): a sink of score 0 without a value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1) if window > 0 else 0
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = max(s.max(), 0.0)
            e = np.exp(s - m)
            out[i, h] = (e @ v[lo:i + 1, g]) / (np.exp(-m) + e.sum())
    return out


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def mingru_scan(z, u, state):
    """z, u [T, W]; state [W].  S_t = (1 - z_t) S_(t-1) + z_t c_t with c = u + 1/2 for u >= 0 and sigmoid(u) below."""
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    out = np.zeros_like(z)
    s = state.copy()
    for t in range(z.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        out[t] = s
    return out, s


def relu_squared(x):
    return np.square(np.maximum(x, 0.0))


# ---- the model ----------------------------------------------------------------------------------------------------
def attention_mixer(h, w: Dict[str, np.ndarray], p: str, m: dict, positions, v_first, is_first_vmix: bool):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, positions, rot["dims"], rot["base"])
        k = rotate_pairs(k, positions, rot["dims"], rot["base"])
    if m.get("v_mix") and not is_first_vmix:
        lam = float(w[p + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    window = (m.get("mask") or {}).get("size", 0)
    o = window_sink_attention(q, k, v, m["scale"], window)
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"], v


def mingru_mixer(h, w, p: str, state):
    z = sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    s, last = mingru_scan(z, u, state)
    g = h @ w[p + "g"].T
    return (s * (g * sigmoid(g))) @ w[p + "o"].T, last


def dense_mlp(h, w, p: str):
    return relu_squared(h @ w[p + "up"].T + w[p + "up.b"]) @ w[p + "down"].T + w[p + "down.b"]


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: List[int], return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence from position 0 (and the residual stream after every layer)."""
    big = cfg["embedding"]["bigram"]
    x = bigram_embedding(tokens, w["embed"], w["bigram"], big["buckets"], big["mul_prev"], big["mul_cur"])
    groups, eps = cfg["norm"]["groups"], cfg["norm"]["eps"]
    positions = np.arange(len(tokens))
    v_first = None
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = group_rmsnorm(x, w[p + "norm1"], groups, eps)
        if layer["type"] == "attention":
            m = layer["mixer"]
            first = bool(m.get("v_mix")) and v_first is None
            y, v = attention_mixer(h, w, p + "mix.", m, positions, v_first, first)
            if first:
                v_first = v
        elif layer["type"] == "mingru":
            y, _ = mingru_mixer(h, w, p + "mix.", np.zeros(layer["mixer"]["width"]))
        else:
            raise ValueError(layer["type"])
        x = x + group_rmsnorm(y, w[p + "norm1b"], groups, eps)
        if layer.get("mlp") is not None:
            h = group_rmsnorm(x, w[p + "norm2"], groups, eps)
            x = x + group_rmsnorm(dense_mlp(h, w, p + "mlp."), w[p + "norm2b"], groups, eps)
        layers.append(x.copy())
    logits = group_rmsnorm(x, w["final.norm"], groups, eps) @ w["head"].T
    return (logits, np.stack(layers)) if return_layers else logits
