"""Bigerax: a decoder of windowed sink-attention layers and minGRU layers between sandwich norms, laid out from parts.

Embedding: token row + hashed (previous token, token) row.  A layer: ``x += post1(mixer(pre1(x)))`` then, if it has a
feed-forward, ``x += post2(ffn(pre2(x)))``, every norm an RMS norm in groups.  Mixers: ``sink_attention`` (grouped
heads, keys and values of different sizes, rotation of adjacent pairs, sliding window, a softmax sink, values mixed
with those of the first such layer) or ``mingru``.  Feed-forward: two matrices with biases around a squared relu.
Then the final norm and the head.  Tensor names: ``embed``, ``bigram``, ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.

This module only *describes* the model; it holds no arithmetic.
"""
from __future__ import annotations

from ..config.bigerax_config import ARCHITECTURE, BigeraxConfig, parse_bigerax_config
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture


def build_spec(cfg: BigeraxConfig) -> ModelSpec:
    d = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("group_rmsnorm", {"width": d, "eps": cfg.norm_eps, "groups": cfg.norm_groups, "weight": name}, category="norm")

    layers = []
    seen_v_mix = False
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            v_mix = None
            if m.v_mix:
                v_mix = "mix" if seen_v_mix else "source"
                seen_v_mix = True
            position = PartSpec("rotary_pairs", {"base": m.rot_base, "dims": m.rot_dims}) if m.rot_dims else None
            mixer = PartSpec("sink_attention", {
                "hidden": d, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim,
                "window": m.window, "scale": m.scale, "sink": True, "bias": True, "bias_suffix": ".b", "position": position,
                "v_mix": v_mix, "v_mix_key": "first", "q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "mix": "mix.vmix"})
        else:
            mixer = PartSpec("mingru", {"hidden": d, "width": m.width, "z": "mix.z", "x": "mix.x", "g": "mix.g", "o": "mix.o",
                                        "z_bias": "mix.z.b", "x_bias": "mix.x.b"})
        extras = {"mixer_post_norm": norm("norm1b")}
        if layer.mlp is not None:
            ffn = PartSpec("dense_mlp", {"hidden": d, "ff": layer.mlp.ff, "activation": "relu2", "bias": True, "bias_suffix": ".b",
                                         "up": "mlp.up", "down": "mlp.down"})
            ffn_norm = norm("norm2")
            extras["ffn_post_norm"] = norm("norm2b")
        else:
            ffn, ffn_norm = PartSpec("none", {}), PartSpec("none", {})
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("sandwich_norm", {}), mixer=mixer, feed_forward=ffn,
                                mixer_norm=norm("norm1"), ffn_norm=ffn_norm, extras=extras))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("bigram_embedding", {"vocab": cfg.vocab, "width": d, "buckets": cfg.buckets, "mul_prev": cfg.mul_prev,
                                                "mul_cur": cfg.mul_cur, "weight": "embed", "pairs": "bigram"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab": cfg.vocab, "width": d, "weight": "head", "tied_to": None}),
        eos_token_ids=cfg.eos_token_ids)


register_architecture(ARCHITECTURE, parse_bigerax_config, build_spec)
