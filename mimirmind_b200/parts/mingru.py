"""minGRU mixer: a gated recurrence whose gates read only the current token.

``z = sigmoid(h·W_zᵀ + b_z)``, ``u = h·W_xᵀ + b_x``, candidate ``c = u + 1/2`` where ``u ≥ 0`` and ``sigmoid(u)`` below;
``S_t = (1 − z)·S_(t−1) + z·c`` element by element; output ``(S_t · silu(h·W_gᵀ))·W_oᵀ``.  The state starts at zero,
is fp32 and is carried per request in the engine's state slots.  The three input projections are one product with an
fp32 result; everything between it and the output projection is fp32 (``csrc/mingru.cu``).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import MIXERS
from .base import LayerCache, Mixer, Runtime, StateSpec, StepContext, WeightView
from .chunks import token_chunks
from .linear import linear

CHUNK = 64               # tokens per chunk of the three-pass scan
CHUNKED_FROM = 256       # a step whose longest portion has at least this many tokens takes the three-pass scan


@MIXERS.register("mingru")
class MinGRU(Mixer):
    """spec params: hidden, width, and the tensor names z, x, g, o (weights), z_bias, x_bias."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, w = spec["hidden"], spec["width"]
        return [TensorSpec(prefix + spec["z"], (w, d)), TensorSpec(prefix + spec["z_bias"], (w,), role="bias"),
                TensorSpec(prefix + spec["x"], (w, d)), TensorSpec(prefix + spec["x_bias"], (w,), role="bias"),
                TensorSpec(prefix + spec["g"], (w, d)), TensorSpec(prefix + spec["o"], (d, w))]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden, self.width = int(spec["hidden"]), int(spec["width"])
        ws = [weights.take(spec[n]) for n in ("z", "x", "g")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.w_zxg = torch.cat(ws, dim=0).contiguous()
        del ws
        bz, bx = weights.take(spec["z_bias"]), weights.take(spec["x_bias"])
        self.b_zx = torch.cat([bz.float(), bx.float()]).contiguous()       # added inside the scan kernels, in fp32
        self.w_o = weights.take(spec["o"]).contiguous()

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.width,), torch.float32)

    @staticmethod
    def _chunks(ctx: StepContext):
        """The step's tokens cut into chunks, per request in order, made once per step."""
        return token_chunks(ctx, CHUNK)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        n = x.shape[0]
        a = linear(x, self.w_zxg, None, self.rt, out_dtype=torch.float32)
        y = torch.empty((n, self.width), dtype=self.rt.dtype, device=a.device)
        # the 32-bit path keeps one order of operations whatever the cutting: it always walks
        if ctx.max_q_len >= CHUNKED_FROM and self.rt.dtype != torch.float32:
            chunk_meta, req_chunks = self._chunks(ctx)
            ops.mingru_chunked(a, y, cache.state, chunk_meta, req_chunks, ctx.state_slots, ctx.positions, self.b_zx)
        else:
            ops.mingru_walk(a, y, cache.state, ctx.req_meta, ctx.state_slots, ctx.positions, ctx.n_requests, self.b_zx)
        return linear(y, self.w_o, None, self.rt)
