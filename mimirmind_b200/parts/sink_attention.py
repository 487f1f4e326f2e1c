"""Windowed self-attention with a softmax sink, keys and values of different sizes, and value mixing between layers.

``q, k, v = h·Wᵀ + b`` with ``H`` query heads and ``G`` key/value heads (query head ``h`` reads key/value head
``h // (H/G)``), keys of size ``key_dim`` and values of size ``value_dim``.  The position encoding turns q and k.
``s = (q·k)·scale``; a query at position ``a`` sees keys ``max(0, a+1−W) .. a``; the weights are
``exp(s_j) / (sink + Σ exp(s_i))`` with ``sink`` 1 (a key of score 0 without a value) or 0 (plain softmax).

Value mixing (``v_mix``): the first layer of a model that names a mixing key is the *source*; every later layer of
that key caches and uses ``(1 − λ)·v + λ·v_source`` of the same token, λ a scalar tensor of the layer.  The source's
values of the step's tokens are handed on through the step context, so nothing of it is cached twice.

Three further options, each a parameter.  A *learned sink*: ``sink`` names a tensor with one logit per head, and the
denominator holds ``exp(logit_h)`` instead of 1.  A *distance bias*: ``distance_bias = {"table", "far", "rows"}`` names a
tensor ``[rows, heads]`` (``rows`` absent: as many as the checkpoint's table has) that is added, unscaled, to the scaled score of a key ``n`` tokens back, at row ``n`` for
``n < rows/2`` and beyond that at rows spaced evenly in ``ln n`` up to ``far``:
``min(rows − 1, rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) · (rows − rows/2)))``; it is unrolled at load into a
table by distance whose last row stands for every larger distance.  An *output gate*: ``gate`` names a projection, and the
joined heads are multiplied by ``sigmoid(h·W_gᵀ)`` before the output projection.

Every size and constant is a parameter; the pools are per-token arrays ``k`` ``(G, key_dim)`` and ``v``
``(G, value_dim)`` of the paged cache.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import CacheArray, KVCacheSpec, LayerCache, Mixer, Runtime, StepContext, WeightView
from .linear import linear


def distance_rows(rows: int, far: float) -> List[int]:
    """Row of the bias table for every distance 0 .. ceil(far): one row per distance below ``rows // 2``, then rows
    spaced evenly in the logarithm of the distance up to ``far``; the last entry (distance >= far) is the last row."""
    half = rows // 2
    if half < 1 or far <= half:
        raise ValueError(f"distance bias: {rows} rows need far > {half}, got {far}")
    out = []
    for n in range(int(math.ceil(far)) + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


@MIXERS.register("sink_attention")
class SinkAttention(Mixer):
    """spec params: hidden, num_heads, num_kv_heads, key_dim, value_dim, window (0: all), scale, sink (bool, or the
    name of a tensor of learned logits), bias (bool: q, k, v and o), position (PartSpec or None), v_mix (None, "source"
    or "mix"), v_mix_key, distance_bias (None or {"table", "far", "rows"}), gate (None or a tensor name), and the
    tensor names q, k, v, o (weights; biases are the name + ``bias_suffix``) and mix (the scalar λ)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, H, G, dk, dv = spec["hidden"], spec["num_heads"], spec["num_kv_heads"], spec["key_dim"], spec["value_dim"]
        out = [TensorSpec(prefix + spec["q"], (H * dk, d)), TensorSpec(prefix + spec["k"], (G * dk, d)),
               TensorSpec(prefix + spec["v"], (G * dv, d)), TensorSpec(prefix + spec["o"], (d, H * dv))]
        if spec.get("bias", False):
            sfx = spec.get("bias_suffix", ".b")
            out += [TensorSpec(prefix + spec["q"] + sfx, (H * dk,), role="bias"), TensorSpec(prefix + spec["k"] + sfx, (G * dk,), role="bias"),
                    TensorSpec(prefix + spec["v"] + sfx, (G * dv,), role="bias"), TensorSpec(prefix + spec["o"] + sfx, (d,), role="bias")]
        if spec.get("v_mix"):
            out.append(TensorSpec(prefix + spec["mix"], (), role="mix"))
        if isinstance(spec.get("sink"), str):
            out.append(TensorSpec(prefix + spec["sink"], (H,), role="bias"))
        if spec.get("distance_bias"):
            # rows None: the checkpoint's table decides how many rows there are
            out.append(TensorSpec(prefix + spec["distance_bias"]["table"], (spec["distance_bias"].get("rows") or -1, H), role="bias"))
        if spec.get("gate"):
            out.append(TensorSpec(prefix + spec["gate"], (H * dv, d)))
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden = int(spec["hidden"])
        self.num_heads, self.num_kv_heads = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.key_dim, self.value_dim = int(spec["key_dim"]), int(spec["value_dim"])
        self.window = int(spec.get("window", 0) or 0)
        self.scale = float(spec["scale"])
        sink = spec.get("sink", True)
        self.sink = bool(sink)
        self.sink_logit = weights.take(sink).float().contiguous() if isinstance(sink, str) else None
        self.dist_bias = None
        db = spec.get("distance_bias")
        if db:
            table = weights.take(db["table"]).float()
            rows = torch.tensor(distance_rows(int(table.shape[0]), float(db["far"])), dtype=torch.long, device=table.device)
            self.dist_bias = table[rows].t().contiguous()        # [heads, ceil(far) + 1]: a head's bias by distance
        self.w_gate = weights.take(spec["gate"]).contiguous() if spec.get("gate") else None
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        pos_spec: Optional[PartSpec] = spec.get("position")
        self.position = POSITION_ENCODINGS.get(pos_spec.kind)(pos_spec, weights, rt) if pos_spec is not None else None
        if self.position is not None and not hasattr(self.position, "pair_rotation"):
            raise ValueError(f"sink attention: the position encoding '{pos_spec.kind}' does not rotate adjacent pairs")
        self.rot_dims, self.inv_freq = self.position.pair_rotation() if self.position is not None else (0, None)
        self.rot_key = ("rope_pairs", self.rot_dims, float(pos_spec["base"])) if self.rot_dims else None
        if self.rot_dims > self.key_dim:
            raise ValueError("sink attention: more rotated dimensions than the key size")
        sfx = spec.get("bias_suffix", ".b")
        ws = [weights.take(spec[n]) for n in ("q", "k", "v")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.w_qkv = torch.cat(ws, dim=0).contiguous()
        del ws
        self.b_qkv = self.b_o = None
        if spec.get("bias", False):
            bs = [weights.take(spec[n] + sfx) for n in ("q", "k", "v")]
            self.b_qkv = torch.cat([b.to(self.w_qkv.dtype) for b in bs], dim=0).contiguous()
            self.b_o = weights.take(spec["o"] + sfx).contiguous()
        self.w_o = weights.take(spec["o"]).contiguous()
        self.v_mix = spec.get("v_mix") or None
        if self.v_mix not in (None, "source", "mix"):
            raise ValueError("sink attention: v_mix is None, 'source' or 'mix'")
        self.v_mix_key = ("v_source", spec.get("v_mix_key", "v"))
        self.mix = 0.0
        if self.v_mix:
            lam = weights.take(spec["mix"])
            # read once at load: the kernel takes it by value (fp32)
            self.mix = float(lam.float().item()) if self.v_mix == "mix" else 0.0

    def kv_cache_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(self.num_kv_heads, self.key_dim, self.window,
                           arrays=(CacheArray("k", (self.num_kv_heads, self.key_dim)), CacheArray("v", (self.num_kv_heads, self.value_dim))))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        n = x.shape[0]
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        k_pages, v_pages = (cache.arrays["k"], cache.arrays["v"]) if cache.writes else (None, None)
        qkv = linear(x, self.w_qkv, self.b_qkv, self.rt)
        q = torch.empty((n, H * dk), dtype=self.rt.dtype, device=qkv.device)
        mode, v_first = 0, None
        if self.v_mix == "source":
            mode = 1
            v_first = ctx.derived[self.v_mix_key] = torch.empty((n, G * dv), dtype=self.rt.dtype, device=qkv.device)
        elif self.v_mix == "mix":
            mode = 2
            v_first = ctx.derived.get(self.v_mix_key)
            if v_first is None:
                raise RuntimeError("sink attention: a layer mixes values before any layer of its key has made them")
        # rotation factors and cache places are the same in every layer that shares them: made once per step
        rot = slots = None
        if self.rot_dims:
            if self.rot_key not in ctx.derived:
                ctx.derived[self.rot_key] = ops.rope_pairs_table(ctx.positions, self.inv_freq, self.rot_dims)
            rot = ctx.derived[self.rot_key]
        if k_pages is not None:
            skey = ("slots", cache.block_table.data_ptr(), cache.page_size)
            if skey not in ctx.derived:
                ctx.derived[skey] = ops.slot_mapping(ctx.positions, ctx.token_req, cache.block_table, cache.page_size)
            slots = ctx.derived[skey]
        ops.qkv_pairs_post(qkv, q, k_pages, v_pages, v_first, rot, slots, cache.page_size, H, G, dk, dv, self.rot_dims, mode, self.mix)
        out = torch.empty((n, H * dv), dtype=self.rt.dtype, device=qkv.device)
        from ..kernels import attention as attn_kernels
        attn_kernels.paged_sink_attention(q, cache, out, ctx, H, G, dk, dv, self.window, self.scale, self.sink,
                                          sink_logit=self.sink_logit, dist_bias=self.dist_bias)
        if self.w_gate is not None:
            gate = linear(x, self.w_gate, None, self.rt)
            out = ops.gated_group_norm(out, 1, H * dv, self.rt.dtype, normalize=False, gate=gate, activation="sigmoid")
        return linear(out, self.w_o, self.b_o, self.rt)
