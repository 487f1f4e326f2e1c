"""Small Bigerax configurations and weights for the tests.  The tensor list is derived here from the configuration
(the names a checkpoint of the design uses), independently of the package's own list."""
import json
import os

import numpy as np


def attention(heads, kv_heads, dim, vdim, window=None, rot=None, scale=None, v_mix=False, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
         "v_mix": v_mix}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def mingru(width, ff=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(vocab, width, groups, eps, buckets, mul_prev, mul_cur, layers):
    return {"architecture": "Bigerax", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": layers}


CONFIGS = {
    # a recurrent layer first, grouped heads, part of the head rotated, a layer without a window or rotation or mixing,
    # keys wider and narrower than values, a layer without a feed-forward, four norm groups
    "P": config(101, 64, 4, 1e-5, 37, 7, 13, [
        mingru(48, ff=80),
        attention(4, 2, 24, 16, window=19, rot=(12, 10000.0), scale=0.31, v_mix=True, ff=96),
        attention(2, 1, 16, 40, v_mix=False, scale=0.4),
        attention(4, 2, 24, 16, window=33, rot=(24, 300.0), v_mix=True, ff=72),
        mingru(32),
    ]),
    # one norm group, a width that the weight-streaming product of a few rows takes, keys and values of one size, one kv head
    "Q": config(320, 256, 1, 1e-6, 64, 3, 5, [
        attention(4, 1, 64, 64, window=50, rot=(64, 250000.0), v_mix=True, ff=256),
        mingru(256, ff=512),
        attention(4, 1, 64, 64, window=50, rot=(64, 250000.0), v_mix=True),
    ]),
    # sizes that fit no tile: odd width per group, odd key size with an even rotated part, a vocabulary of 77
    "R": config(77, 54, 3, 1e-6, 11, 1, 1, [
        attention(3, 3, 9, 7, window=8, rot=(6, 100.0), v_mix=False, ff=33),
        mingru(21, ff=17),
        attention(6, 2, 10, 12, window=70, rot=(10, 10000.0), v_mix=True, ff=40),
        attention(6, 2, 10, 12, window=16, rot=(4, 10000.0), v_mix=True),
    ]),
    # key and value sizes of the tensor-core attention kernels, keys wider and narrower than values, windows that are
    # and are not multiples of a key tile, eight query heads on two kv heads
    "S": config(200, 128, 2, 1e-6, 97, 5, 3, [
        attention(4, 2, 32, 64, window=64, rot=(32, 10000.0), v_mix=True, ff=192),
        attention(8, 2, 96, 32, window=45, rot=(64, 250000.0), v_mix=False, ff=128),
        mingru(96),
        attention(4, 2, 32, 64, window=130, rot=(16, 10000.0), v_mix=True),
    ]),
}
LENGTHS = {"P": [1, 9, 77, 300], "Q": [5, 70, 280], "R": [2, 33, 150, 270], "S": [3, 64, 129, 290]}


def tensor_shapes(cfg):
    d, v = cfg["width"], cfg["vocab"]
    out = {"embed": (v, d), "bigram": (cfg["embedding"]["bigram"]["buckets"] + 1, d), "final.norm": (d,), "head": (v, d)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = out[p + "norm1b"] = (d,)
        if layer["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * dk, d), p + "mix.q.b": (H * dk,), p + "mix.k": (G * dk, d), p + "mix.k.b": (G * dk,),
                        p + "mix.v": (G * dv, d), p + "mix.v.b": (G * dv,), p + "mix.o": (d, H * dv), p + "mix.o.b": (d,)})
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()
        else:
            w = m["width"]
            out.update({p + "mix.z": (w, d), p + "mix.z.b": (w,), p + "mix.x": (w, d), p + "mix.x.b": (w,), p + "mix.g": (w, d),
                        p + "mix.o": (d, w)})
        if layer["mlp"] is not None:
            f = layer["mlp"]["ff"]
            out.update({p + "norm2": (d,), p + "norm2b": (d,), p + "mlp.up": (f, d), p + "mlp.up.b": (f,), p + "mlp.down": (d, f),
                        p + "mlp.down.b": (d,)})
    return out


def random_weights(cfg, seed, gain=1.0):
    """Weights large enough that every mechanism moves the logits: matrices ~ N(0, gain / sqrt(in)), biases ~ 0.1 N, norm
    weights ~ 1 + 0.1 N, mixing weights in (0.2, 0.8)."""
    rng = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("vmix"):
            w = np.asarray(rng.uniform(0.2, 0.8))
        elif "norm" in name:
            w = 1.0 + 0.1 * rng.randn(*shape)
        elif name.endswith(".b"):
            w = 0.1 * rng.randn(*shape)
        elif name in ("embed", "bigram"):
            w = rng.randn(*shape) * (1.0 if name == "embed" else 0.5)
        else:
            w = rng.randn(*shape) * gain / np.sqrt(shape[1])
        out[name] = w.astype(np.float32)
    return out


def write_model(folder, cfg, seed, gain=1.0, overrides=None):
    """config.json + model.safetensors (bfloat16) in ``folder``."""
    import torch
    from mimirmind_b200.weights.safetensors_io import write_safetensors
    w = random_weights(cfg, seed, gain)
    w.update(overrides or {})
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: torch.from_numpy(np.asarray(v)).to(torch.bfloat16) for k, v in w.items()})
    return folder
