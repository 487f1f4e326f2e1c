"""Two mixers side by side on the same input: each output is RMS-normed over the model width with a plain weight of its
own, and the mixer's result is ``scale`` times their sum (one half: the mean).

The two sides are built from their own part specs through the mixer registry, so any pair of registered mixers can stand
here; a side that keeps keys and values and a side that keeps a state share the layer's cache entry (the paged arrays go
to the one, the state slot to the other).  Two sides of the same kind of memory are refused.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import MIXERS
from .base import KVCacheSpec, LayerCache, Mixer, Runtime, StateSpec, StepContext, WeightView


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    """spec params: hidden, eps, scale, left and right (PartSpecs of mixers), left_out and right_out (names of the two
    norm weights)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        out = []
        for side in ("left", "right"):
            out += MIXERS.get(spec[side].kind).tensor_specs(spec[side], prefix)
            out.append(TensorSpec(prefix + spec[side + "_out"], (spec["hidden"],), role="norm"))
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden, self.eps, self.scale = int(spec["hidden"]), float(spec["eps"]), float(spec.get("scale", 0.5))
        self.left = MIXERS.get(spec["left"].kind)(spec["left"], weights, rt)
        self.right = MIXERS.get(spec["right"].kind)(spec["right"], weights, rt)
        self.w_left = weights.take(spec["left_out"]).float().contiguous()
        self.w_right = weights.take(spec["right_out"]).float().contiguous()
        if self.left.kv_cache_spec() is not None and self.right.kv_cache_spec() is not None:
            raise ValueError("parallel mixers: both sides keep a paged cache; a layer has one")
        if self.left.state_spec() is not None and self.right.state_spec() is not None:
            raise ValueError("parallel mixers: both sides keep a state; a layer has one")

    def kv_cache_spec(self) -> Optional[KVCacheSpec]:
        return self.left.kv_cache_spec() or self.right.kv_cache_spec()

    def state_spec(self) -> Optional[StateSpec]:
        return self.left.state_spec() or self.right.state_spec()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        a = self.left.forward(x, ctx, cache)
        b = self.right.forward(x, ctx, cache)
        return ops.normed_mean2(a, b, self.w_left, self.w_right, self.eps, self.scale)
