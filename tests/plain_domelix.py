"""Plain, slow implementation of the Domelix decoder in numpy float64: whole sequences, no cache, one function per
mechanism.  It is the oracle of the Domelix tests and shares no code with the package.

Notation: ``T`` tokens, width ``D``; a linear map stored ``[out, in]`` is applied as ``x @ W.T``.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np


# ---- container --------------------------------------------------------------------------------------------------
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
        raw, shape, dt = data[lo:hi], tuple(info["shape"]), info["dtype"]
        if dt == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            out[name] = u.view(np.float32).astype(np.float64).reshape(shape)
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


# ---- small functions ----------------------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


# ---- mechanisms ---------------------------------------------------------------------------------------------------
def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance table for a key ``n`` tokens back: one row per distance below ``rows/2``, then rows spaced
    evenly in ln(distance) up to ``far``, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def biased_sink_attention_core(q, k, v, rel, sink, scale, far, positions=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]: causal softmax over all earlier tokens with a bias per (distance row, head)
    added to the scaled score and exp(sink_h) in the denominator only.  Returns [T, H, dv]."""
    T, heads, _ = q.shape
    kv_heads, vdim = k.shape[1], v.shape[2]
    rows = rel.shape[0]
    out = np.zeros((T, heads, vdim))
    per = heads // kv_heads
    for hd in range(heads):
        g = hd // per
        for i in range(T):
            s = np.array([q[i, hd] @ k[j, g] * scale + rel[distance_bucket(i - j, rows, far), hd] for j in range(i + 1)])
            m = max(s.max(), sink[hd])
            e = np.exp(s - m)
            out[i, hd] = (e / (e.sum() + math.exp(sink[hd] - m))) @ v[: i + 1, g]
    return out


def biased_sink_attention(h, wq, wk, wv, wg, wo, rel, sink, heads, kv_heads, dim, vdim, scale, far):
    """Grouped heads, no rotation, a learned distance bias, a learned sink, and a sigmoid gate on the joined heads."""
    T = h.shape[0]
    q = (h @ wq.T).reshape(T, heads, dim)
    k = (h @ wk.T).reshape(T, kv_heads, dim)
    v = (h @ wv.T).reshape(T, kv_heads, vdim)
    out = biased_sink_attention_core(q, k, v, rel, sink, scale, far)
    joined = out.reshape(T, heads * vdim) * sigmoid(h @ wg.T)
    return joined @ wo.T


def decayed_outer_products(q, k, v, decay, state=None):
    """Per head S_t = decay * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, dk], v [T, H, dv], decay [H]."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = np.zeros((H, dk, dv)) if state is None else state.copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hd in range(H):
            S[hd] = decay[hd] * S[hd] + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    return o, S


def lightning(h, wq, wk, wv, wg, wo, norm_w, decay, heads, dim, vdim, eps):
    T = h.shape[0]
    q = silu(h @ wq.T).reshape(T, heads, dim)
    k = silu(h @ wk.T).reshape(T, heads, dim)
    v = silu(h @ wv.T).reshape(T, heads, vdim)
    o, _ = decayed_outer_products(q, k, v, np.asarray(decay, dtype=np.float64))
    y = rms(o.reshape(T, heads * vdim), eps) * norm_w * sigmoid(h @ wg.T)
    return y @ wo.T


def parallel_mixer(h, w: Dict[str, np.ndarray], m: dict, eps: float):
    """Two mixers on the same input; each output is RMS-normed over the width with a plain weight, and the two are averaged."""
    L, R = m["left"], m["right"]
    left = biased_sink_attention(h, w["left.q"], w["left.k"], w["left.v"], w["left.g"], w["left.o"], w["left.rel"], w["left.sink"],
                                 L["heads"], L["kv_heads"], L["dim"], L["vdim"], L["scale"], L["bias_max"])
    right = lightning(h, w["right.q"], w["right.k"], w["right.v"], w["right.g"], w["right.o"], w["right.norm"], R["decay"],
                      R["heads"], R["dim"], R["vdim"], eps)
    return 0.5 * (rms(left, eps) * w["left.out"] + rms(right, eps) * w["right.out"])


def causal_conv(x, taps):
    """x [T, C], taps [C, K]: y_t = sum_j taps[:, K-1-j] * x_(t-j), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = np.zeros_like(x)
    for t in range(T):
        for j in range(K):
            if t - j >= 0:
                y[t] += taps[:, K - 1 - j] * x[t - j]
    return y


def gated_delta(h, w: Dict[str, np.ndarray], m: dict, eps: float):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).reshape(T, G, dk)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).reshape(T, G, dk)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w["b"].T)
    g = np.exp(-np.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))
    per = H // G
    S = np.zeros((H, dk, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hd in range(H):
            kk, qq = k[t, hd // per], q[t, hd // per]
            S[hd] = g[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ kk)
            S[hd] = S[hd] + np.outer(kk, u)
            o[t, hd] = S[hd].T @ qq
    y = rms(o, eps) * w["norm"] * silu(h @ w["g"].T).reshape(T, H, dv)
    return y.reshape(T, H * dv) @ w["o"].T


def rotate_half(x, positions, dims, base):
    """x [T, H, d]: dimension i < dims/2 is paired with i + dims/2 and the pair turned by position * base^(-2i/dims)."""
    half = dims // 2
    out = x.copy()
    f = base ** (-2.0 * np.arange(half) / dims)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def retention(h, w: Dict[str, np.ndarray], m: dict, eps: float, positions=None):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    positions = np.arange(T) if positions is None else positions
    q = (h @ w["q"].T).reshape(T, H, dk)
    k = (h @ w["k"].T).reshape(T, H, dk)
    v = (h @ w["v"].T).reshape(T, H, dv)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = rotate_half(q, positions, rot["dims"], rot["base"])
        k = rotate_half(k, positions, rot["dims"], rot["base"])
    k = k * dk ** -0.5
    o, _ = decayed_outer_products(q, k, v, np.asarray(m["decay"], dtype=np.float64))
    y = rms(o, eps).reshape(T, H * dv) * silu(h @ w["g"].T)
    return y @ w["o"].T


def route(z, top: int, groups: int, keep: int):
    """z [T, E] router logits -> (chosen experts [T, top], their weights [T, top]).  Softmax over all experts; experts
    in ``groups`` equal runs of neighbours, a run scored by its best expert, only the ``keep`` best runs eligible."""
    T, E = z.shape
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s = s / s.sum(axis=-1, keepdims=True)
    idx = np.zeros((T, top), dtype=np.int64)
    wts = np.zeros((T, top))
    size = E // groups
    for t in range(T):
        gs = s[t].reshape(groups, size).max(axis=-1)
        best = np.argsort(-gs, kind="stable")[:keep]
        allowed = np.zeros(E, dtype=bool)
        for g in best:
            allowed[g * size:(g + 1) * size] = True
        masked = np.where(allowed, s[t], -1.0)
        chosen = np.argsort(-masked, kind="stable")[:top]
        idx[t] = chosen
        wts[t] = s[t, chosen] / (s[t, chosen].sum() + 1e-20)
    return idx, wts


def mixture_of_experts(h, w: Dict[str, np.ndarray], mlp: dict):
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    idx, wts = route(h @ w["router"].T, r["top"], groups["count"], groups["keep"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t], wts[t]):
            x = h[t]
            out[t] += a * ((silu(x @ w[f"e{e}.gate"].T) * (x @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T)
    return out


# ---- the model -----------------------------------------------------------------------------------------------------
def _sub(weights: Dict[str, np.ndarray], prefix: str) -> Dict[str, np.ndarray]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def mixer(kind: str, h, w, m, eps):
    if kind == "parallel":
        return parallel_mixer(h, w, m, eps)
    if kind == "delta":
        return gated_delta(h, w, m, eps)
    if kind == "retention":
        return retention(h, w, m, eps)
    raise ValueError(kind)


def forward(cfg: dict, weights: Dict[str, np.ndarray], tokens: List[int], layers_out: Optional[list] = None) -> np.ndarray:
    """Logits [T, vocab] of one whole sequence; ``layers_out`` collects the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = weights["embed"][np.asarray(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a = mixer(layer["type"], norm_one_plus(x, weights[p + "norm1"], eps), _sub(weights, p + "mix."), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            a = a + mixture_of_experts(norm_one_plus(x, weights[p + "norm2"], eps), _sub(weights, p + "mlp."), layer["mlp"])
        x = x + a
        if layers_out is not None:
            layers_out.append(x.copy())
    return norm_one_plus(x, weights["final.norm"], eps) @ weights["head"].T
