"""Small Domelix configurations and weights for the tests.  The tensor list is derived here from the configuration
(the names a checkpoint of the design uses), independently of the package's own list."""
import json
import os

import numpy as np


def moe(ff, experts, top, groups=None):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def parallel(left, right, mlp=None):
    """left: (heads, kv_heads, dim, vdim, scale, bias_max, bias_rows); right: (heads, dim, vdim, decay list)"""
    H, G, dk, dv, scale, far, rows = left
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": scale, "bias_max": far, "bias_rows": rows},
                      "right": {"heads": right[0], "dim": right[1], "vdim": right[2], "decay": list(right[3])}}}


def delta(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def retention(heads, dim, vdim, decay, rot=None, mlp=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "retention", "mixer": m, "mlp": mlp}


def config(vocab, width, eps, layers):
    return {"architecture": "Domelix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # a parallel layer first, grouped heads everywhere, keys wider and narrower than values, part of the head rotated,
    # three taps, a layer without a feed-forward, experts in three groups of which two are kept
    "P": config(101, 64, 1e-5, [
        parallel((4, 2, 24, 16, 0.3, 37, 10), (3, 16, 8, (0.5, 0.9, 0.99)), moe(40, 6, 2, (3, 2))),
        delta(4, 2, 16, 24, 3, moe(24, 4, 1)),
        retention(2, 24, 16, (0.97, 0.8), rot=(12, 100.0), mlp=moe(40, 6, 2, (3, 2))),
        parallel((2, 1, 16, 40, 0.25, 50, 8), (2, 8, 16, (0.7, 0.995))),
        delta(2, 2, 8, 8, 4),
    ]),
    # sizes the tensor-core kernels take (attention 64/64 and 96/32, expert products with depths that are multiples of 8), a
    # width that the weight-streaming product of a few rows takes, whole heads rotated, one group of experts
    "Q": config(320, 256, 1e-6, [
        delta(4, 4, 64, 64, 4, moe(64, 8, 3)),
        parallel((8, 2, 64, 64, 0.125, 300, 32), (4, 64, 32, (0.6, 0.9, 0.97, 0.999)), moe(64, 8, 3)),
        retention(2, 128, 32, (0.98, 0.9995), rot=(128, 1000000.0), mlp=moe(128, 4, 2, (2, 1))),
        parallel((4, 1, 96, 32, 0.1, 64, 12), (2, 32, 64, (0.9, 0.99)), moe(64, 8, 3)),
    ]),
    # sizes that fit no tile: odd width, odd key and value sizes, an odd number of bias rows, a bias range that is no whole
    # number, one head, one tap, every expert chosen, a retention layer without rotation, a vocabulary of 77
    "R": config(77, 54, 1e-6, [
        retention(3, 10, 7, (0.9, 0.5, 0.99), mlp=moe(33, 5, 5)),
        parallel((3, 3, 9, 7, 0.33, 20.5, 7), (1, 10, 12, (0.93,)), moe(17, 6, 2, (2, 1))),
        delta(6, 2, 10, 5, 2, moe(33, 5, 5)),
        delta(1, 1, 12, 6, 1),
        parallel((6, 2, 10, 12, 0.3, 130, 16), (5, 6, 3, (0.2, 0.6, 0.9, 0.99, 0.999))),
    ]),
    # no layer keeps keys and values (no page pool at all), a single layer of each remaining kind, one expert of one
    "N": config(90, 48, 1e-5, [
        retention(2, 16, 8, (0.9, 0.99), rot=(16, 50.0), mlp=moe(16, 1, 1)),
        delta(2, 1, 8, 16, 4, moe(16, 3, 2)),
    ]),
}
LENGTHS = {"P": [1, 9, 77, 300], "Q": [5, 70, 280], "R": [2, 33, 150, 270], "N": [3, 40, 290]}


def tensor_shapes(cfg):
    d, v = cfg["width"], cfg["vocab"]
    out = {"embed": (v, d), "final.norm": (d,), "head": (v, d)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (d,)
        if layer["type"] == "parallel":
            L, R = m["left"], m["right"]
            H, G, dk, dv = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
            out.update({p + "mix.left.q": (H * dk, d), p + "mix.left.k": (G * dk, d), p + "mix.left.v": (G * dv, d),
                        p + "mix.left.rel": (L["bias_rows"], H), p + "mix.left.sink": (H,), p + "mix.left.g": (H * dv, d),
                        p + "mix.left.o": (d, H * dv), p + "mix.left.out": (d,), p + "mix.right.out": (d,)})
            H, dk, dv = R["heads"], R["dim"], R["vdim"]
            out.update({p + "mix.right.q": (H * dk, d), p + "mix.right.k": (H * dk, d), p + "mix.right.v": (H * dv, d),
                        p + "mix.right.g": (H * dv, d), p + "mix.right.o": (d, H * dv), p + "mix.right.norm": (H * dv,)})
        elif layer["type"] == "delta":
            H, G, dk, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            out.update({p + "mix.q": (G * dk, d), p + "mix.q.conv": (G * dk, K), p + "mix.k": (G * dk, d), p + "mix.k.conv": (G * dk, K),
                        p + "mix.v": (H * dv, d), p + "mix.v.conv": (H * dv, K), p + "mix.b": (H, d), p + "mix.a": (H, d),
                        p + "mix.A_log": (H,), p + "mix.dt_bias": (H,), p + "mix.norm": (dv,), p + "mix.g": (H * dv, d), p + "mix.o": (d, H * dv)})
        else:
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * dk, d), p + "mix.k": (H * dk, d), p + "mix.v": (H * dv, d), p + "mix.g": (H * dv, d),
                        p + "mix.o": (d, H * dv)})
        if layer["mlp"] is not None:
            f, E = layer["mlp"]["expert"]["ff"], layer["mlp"]["router"]["experts"]
            out[p + "norm2"] = (d,)
            out[p + "mlp.router"] = (E, d)
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (f, d), p + f"mlp.e{e}.up": (f, d), p + f"mlp.e{e}.down": (d, f)})
    return out


def random_weights(cfg, seed, gain=1.0):
    """Weights large enough that every mechanism moves the logits: matrices ~ N(0, gain / sqrt(in)); the norms stored
    around zero ~ 0.1 N; the plain norm weights ~ 1 + 0.1 N; distance tables and sinks ~ N(0, 1); taps ~ 0.5 N; the
    router spread wide, so that a choice of experts is seldom a near tie."""
    rng = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            w = 0.1 * rng.randn(*shape)
        elif leaf in ("out", "norm"):
            w = 1.0 + 0.1 * rng.randn(*shape)
        elif leaf in ("rel", "sink"):
            w = rng.randn(*shape)
        elif leaf == "conv":
            w = 0.5 * rng.randn(*shape)
        elif leaf in ("A_log", "dt_bias"):
            w = 0.5 * rng.randn(*shape)
        elif leaf == "router":
            w = rng.randn(*shape) * 4.0 / np.sqrt(shape[1])
        elif name == "embed":
            w = rng.randn(*shape)
        else:
            w = rng.randn(*shape) * gain / np.sqrt(shape[1])
        out[name] = w.astype(np.float32)
    return out


def write_model(folder, cfg, seed, gain=1.0, overrides=None, keep_rows_key=True):
    """config.json + model.safetensors (bfloat16) in ``folder``; without ``keep_rows_key`` the configuration does not say how
    many rows the distance tables have (the checkpoint's tables decide)."""
    import copy
    import torch
    from mimirmind_b200.weights.safetensors_io import write_safetensors
    w = random_weights(cfg, seed, gain)
    w.update(overrides or {})
    os.makedirs(folder, exist_ok=True)
    written = copy.deepcopy(cfg)
    if not keep_rows_key:
        for layer in written["layers"]:
            if layer["type"] == "parallel":
                del layer["mixer"]["left"]["bias_rows"]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(written, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: torch.from_numpy(np.asarray(v)).to(torch.bfloat16) for k, v in w.items()})
    return folder
