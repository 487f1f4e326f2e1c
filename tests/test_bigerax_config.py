"""Bigerax without a GPU: the configuration reader, the layout of parts, the tensor list, and the plain implementation's
mechanisms against hand-made cases."""
import copy

import numpy as np
import pytest

import bigerax_util as bu
import plain_bigerax as pb


def parse(cfg):
    from mimirmind_b200.registry import get_architecture
    entry = get_architecture("Bigerax")
    parsed = entry.parse_config(cfg, "config.json")
    return parsed, entry.build_spec(parsed)


def test_every_size_and_constant_comes_from_the_file():
    cfg = bu.CONFIGS["P"]
    parsed, spec = parse(cfg)
    assert (spec.vocab_size, spec.hidden_size, len(spec.layers)) == (101, 64, 5)
    assert spec.embedding.kind == "bigram_embedding" and spec.embedding["buckets"] == 37 and spec.embedding["mul_prev"] == 7
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["mingru", "sink_attention", "sink_attention", "sink_attention", "mingru"]
    a1, a2, a3 = spec.layers[1].mixer, spec.layers[2].mixer, spec.layers[3].mixer
    assert (a1["num_heads"], a1["num_kv_heads"], a1["key_dim"], a1["value_dim"], a1["window"], a1["scale"]) == (4, 2, 24, 16, 19, 0.31)
    assert a1["position"].kind == "rotary_pairs" and a1["position"]["dims"] == 12 and a1["position"]["base"] == 10000.0
    assert a2["position"] is None and a2["window"] == 0
    # the first layer that mixes values is the source, later ones mix, a layer that does not say so does neither
    assert (a1["v_mix"], a2["v_mix"], a3["v_mix"]) == ("source", None, "mix")
    assert spec.layers[0].feed_forward.kind == "dense_mlp" and spec.layers[4].feed_forward.kind == "none"
    assert spec.layers[2].feed_forward.kind == "none" and "ffn_post_norm" not in spec.layers[2].extras
    assert all(layer.mixer_norm["groups"] == 4 and layer.mixer_norm["eps"] == 1e-5 for layer in spec.layers)


@pytest.mark.parametrize("name", sorted(bu.CONFIGS))
def test_the_declared_tensors_are_the_checkpoints(name):
    from mimirmind_b200.weights.store import expected_tensors
    _, spec = parse(bu.CONFIGS[name])
    assert {k: tuple(v.shape) for k, v in expected_tensors(spec).items()} == bu.tensor_shapes(bu.CONFIGS[name])


def test_a_checkpoint_that_does_not_fit_is_refused_with_one_message(tmp_path):
    import torch
    from mimirmind_b200.weights.store import WeightsError, load_spec, load_tensors
    cfg = bu.CONFIGS["R"]
    w = bu.random_weights(cfg, 0)
    w["l0.mix.q.b"] = w["l0.mix.q.b"][:-1]
    del w["l1.mix.g"]
    w["l9.extra"] = np.zeros(3, dtype=np.float32)
    folder = bu.write_model(str(tmp_path), cfg, 0, overrides=w)
    # the overrides only replace: drop the deleted one by writing the file again without it
    from mimirmind_b200.weights.safetensors_io import write_safetensors
    write_safetensors(str(tmp_path / "model.safetensors"), {k: torch.from_numpy(np.asarray(v)).to(torch.bfloat16) for k, v in w.items()})
    _, spec = load_spec(folder)
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, spec, torch.float32, "cpu")
    assert "l1.mix.g" in str(e.value) and "l9.extra" in str(e.value) and "l0.mix.q.b" in str(e.value)


@pytest.mark.parametrize("edit,message", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=13), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "layers[1].mixer.scale"),
    (lambda c: c["layers"][0].update(type="lstm"), "lstm"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "moe"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "embedding.bigram.buckets"),
])
def test_a_config_that_cannot_run_names_its_key(edit, message):
    from mimirmind_b200.config.model_config import ConfigError
    cfg = copy.deepcopy(bu.CONFIGS["P"])
    edit(cfg)
    with pytest.raises(ConfigError, match=message.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
        parse(cfg)


def test_cache_groups_and_state_follow_the_layers():
    """What the cache manager is asked for: one group per (kv heads, key and value sizes, window), state for the
    recurrent layers and for the embedding."""
    import torch
    from mimirmind_b200.engine.model import Model
    from mimirmind_b200.parts.base import Runtime
    from mimirmind_b200.weights.store import random_tensors
    _, spec = parse(bu.CONFIGS["P"])
    model = Model(spec, random_tensors(spec, 0, torch.float32, "cpu"), Runtime(torch.float32, torch.device("cpu")))
    groups = {g.name: g for g in model.cache_groups()}
    assert sorted((g.window, g.entries) for g in groups.values()) == [(0, (2,)), (19, (1,)), (33, (3,))]
    g = next(g for g in groups.values() if g.window == 19)
    assert [(n, s) for n, s, _ in g.token_arrays()] == [("k", (2, 24)), ("v", (2, 16))]
    states = model.state_specs()
    assert sorted(states) == [-1, 0, 4] and states[0].shape == (48,) and states[4].shape == (32,) and states[-1].dtype == torch.int32


# ---- the plain implementation's own mechanisms against hand-made cases ----------------------------------------------------
def test_plain_sink_softmax_and_window():
    q = np.zeros((4, 1, 2))
    k = np.zeros((4, 1, 2))
    v = np.arange(4.0).reshape(4, 1, 1) + 1
    # all scores 0: every seen key and the sink weigh the same
    out = pb.window_sink_attention(q, k, v, 1.0, 0)[:, 0, 0]
    assert np.allclose(out, [1 / 2, 3 / 3, 6 / 4, 10 / 5])
    out = pb.window_sink_attention(q, k, v, 1.0, 2)[:, 0, 0]
    assert np.allclose(out, [1 / 2, 3 / 3, 5 / 3, 7 / 3])


def test_plain_group_norm_and_rotation_and_scan():
    x = np.array([[3.0, 4.0, 0.0, 2.0]])
    assert np.allclose(pb.group_rmsnorm(x, np.ones(4), 2, 0.0), [[3 / np.sqrt(12.5), 4 / np.sqrt(12.5), 0.0, np.sqrt(2.0)]])
    r = pb.rotate_pairs(np.array([[[1.0, 0.0, 5.0, 7.0]]]), [1], 2, 10000.0)
    assert np.allclose(r, [[[np.cos(1.0), np.sin(1.0), 5.0, 7.0]]])
    z, u = np.full((3, 1), 0.5), np.array([[1.0], [-30.0], [0.0]])
    out, last = pb.mingru_scan(z, u, np.zeros(1))
    assert np.allclose(out[:, 0], [0.75, 0.375, 0.4375]) and np.allclose(last, 0.4375)
    emb = pb.bigram_embedding([2, 1], np.eye(3), np.arange(15.0).reshape(5, 3), 4, 3, 5)
    assert np.allclose(emb[0], np.eye(3)[2] + [12, 13, 14]) and np.allclose(emb[1], np.eye(3)[1] + [9, 10, 11])     # (2*3 + 1*5) % 4 = 3
