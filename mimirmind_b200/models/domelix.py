"""Domelix: a decoder whose layers run a mixer and a mixture of experts side by side, laid out from parts.

A layer: ``x += mixer(norm1(x)) + experts(norm2(x))``, both norms RMS norms whose weight is stored around zero
(``1 + w`` multiplies).  Mixers, by the layer's ``type``:

* ``parallel``: two mixers on the same input, each output RMS-normed over the width, the two averaged.  Left: causal
  softmax attention with grouped heads, no rotation, a learned bias by (log-spaced) distance, a learned sink per head
  and a sigmoid output gate.  Right: lightning attention, a matrix state per head with a constant decay, silu on q, k
  and v, one RMS norm over the joined heads, a sigmoid gate.
* ``delta``: the gated delta rule: short causal convolutions and silu on q, k and v, q and k of unit length, a learned
  decay and write strength per token and head, an RMS norm per head, a silu gate.
* ``retention``: a matrix state per head with a constant decay, q and k rotated by position (half-split pairs), an
  RMS norm per head without weight, a silu gate.

Feed-forward: routed experts (softmax router, choice limited to the best groups).  Then the final norm and the head.
Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.

This module only *describes* the model; it holds no arithmetic.
"""
from __future__ import annotations

from ..config.domelix_config import ARCHITECTURE, DecayedState, DomelixConfig, parse_domelix_config
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

UNIT_EPS = 1e-6      # inside the root when q and k of the delta rule are brought to unit length


def _decayed_state(d: int, eps: float, m: DecayedState, stem: str, lightning: bool) -> PartSpec:
    """Retention (rotation, k scaled, a norm per head, silu gate) or lightning attention (silu on q, k, v, one norm over
    the joined heads with a weight, sigmoid gate)."""
    common = {"hidden": d, "heads": m.heads, "qk_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "eps": eps, "decay": list(m.decay),
              "delta": None, "conv": 0, "q": stem + "q", "k": stem + "k", "v": stem + "v", "g": stem + "g", "o": stem + "o"}
    if lightning:
        return PartSpec("linear_state", {**common, "activation": "silu", "rotary": None, "unit_eps": None, "out_norm": "all",
                                         "out_weight": stem + "norm", "gate_activation": "sigmoid"})
    return PartSpec("linear_state", {**common, "activation": None, "rotary": {"dims": m.rot_dims, "base": m.rot_base} if m.rot_dims else None,
                                     "unit_eps": None, "k_scale": m.dim ** -0.5, "out_norm": "head", "out_weight": None,
                                     "gate_activation": "silu"})


def build_spec(cfg: DomelixConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": d, "eps": eps, "weight": name, "offset": 1.0}, category="norm")

    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "parallel":
            L = m.left
            left = PartSpec("sink_attention", {
                "hidden": d, "num_heads": L.heads, "num_kv_heads": L.kv_heads, "key_dim": L.dim, "value_dim": L.vdim, "window": 0,
                "scale": L.scale, "sink": "mix.left.sink", "bias": False, "position": None, "v_mix": None,
                "distance_bias": {"table": "mix.left.rel", "far": L.bias_max, "rows": L.bias_rows}, "gate": "mix.left.g",
                "q": "mix.left.q", "k": "mix.left.k", "v": "mix.left.v", "o": "mix.left.o"})
            mixer = PartSpec("parallel_mixers", {"hidden": d, "eps": eps, "scale": 0.5, "left": left,
                                                 "right": _decayed_state(d, eps, m.right, "mix.right.", lightning=True),
                                                 "left_out": "mix.left.out", "right_out": "mix.right.out"})
        elif layer.type == "delta":
            mixer = PartSpec("linear_state", {
                "hidden": d, "heads": m.heads, "qk_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim, "eps": eps, "decay": "learned",
                "delta": "mix.b", "a": "mix.a", "A_log": "mix.A_log", "dt_bias": "mix.dt_bias", "conv": m.conv, "conv_suffix": ".conv",
                "activation": "silu", "rotary": None, "unit_eps": UNIT_EPS, "q_scale": m.dim ** -0.5, "out_norm": "head",
                "out_weight": "mix.norm", "gate_activation": "silu", "q": "mix.q", "k": "mix.k", "v": "mix.v", "g": "mix.g", "o": "mix.o"})
        else:
            mixer = _decayed_state(d, eps, m, "mix.", lightning=False)
        if layer.mlp is not None:
            f = layer.mlp
            ffn = PartSpec("routed_experts", {"hidden": d, "ff": f.ff, "experts": f.experts, "top": f.top, "groups": f.groups, "keep": f.keep,
                                              "router": "mlp.router", "expert": "mlp.e{}"})
            ffn_norm = norm("norm2")
        else:
            ffn, ffn_norm = PartSpec("none", {}), PartSpec("none", {})
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("parallel_branches", {}), mixer=mixer, feed_forward=ffn,
                                mixer_norm=norm("norm1"), ffn_norm=ffn_norm))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "width": d, "scale": 1.0, "weight": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab": cfg.vocab, "width": d, "weight": "head", "tied_to": None}),
        eos_token_ids=cfg.eos_token_ids)


register_architecture(ARCHITECTURE, parse_domelix_config, build_spec)
