"""Domelix without a GPU: the configuration reader, the layout of parts, the tensor list, the table of distance rows, and
the plain implementation's mechanisms against hand-made cases."""
import copy
import math

import numpy as np
import pytest

import domelix_util as du
import plain_domelix as pd


def parse(cfg):
    from mimirmind_b200.registry import get_architecture
    entry = get_architecture("Domelix")
    parsed = entry.parse_config(cfg, "config.json")
    return parsed, entry.build_spec(parsed)


def test_every_size_and_constant_comes_from_the_file():
    parsed, spec = parse(du.CONFIGS["P"])
    assert (spec.vocab_size, spec.hidden_size, len(spec.layers)) == (101, 64, 5)
    assert [layer.mixer.kind for layer in spec.layers] == ["parallel_mixers", "linear_state", "linear_state", "parallel_mixers", "linear_state"]
    assert all(layer.block.kind == "parallel_branches" for layer in spec.layers)
    assert all(layer.mixer_norm["offset"] == 1.0 and layer.mixer_norm["eps"] == 1e-5 for layer in spec.layers)
    par = spec.layers[0].mixer
    left, right = par["left"], par["right"]
    assert left.kind == "sink_attention" and right.kind == "linear_state" and par["scale"] == 0.5
    assert (left["num_heads"], left["num_kv_heads"], left["key_dim"], left["value_dim"], left["scale"], left["window"]) == (4, 2, 24, 16, 0.3, 0)
    assert left["distance_bias"] == {"table": "mix.left.rel", "far": 37, "rows": 10} and left["sink"] == "mix.left.sink" and left["gate"] == "mix.left.g"
    assert left["position"] is None and not left["bias"]
    assert (right["heads"], right["key_dim"], right["value_dim"], right["decay"]) == (3, 16, 8, [0.5, 0.9, 0.99])
    assert right["activation"] == "silu" and right["out_norm"] == "all" and right["gate_activation"] == "sigmoid" and not right["delta"]
    dl = spec.layers[1].mixer
    assert (dl["heads"], dl["qk_heads"], dl["key_dim"], dl["value_dim"], dl["conv"]) == (4, 2, 16, 24, 3)
    assert dl["decay"] == "learned" and dl["delta"] == "mix.b" and dl["unit_eps"] == 1e-6 and dl["q_scale"] == 16 ** -0.5
    ret = spec.layers[2].mixer
    assert ret["rotary"] == {"dims": 12, "base": 100.0} and ret["k_scale"] == 24 ** -0.5 and ret["out_weight"] is None
    assert ret["out_norm"] == "head" and ret["gate_activation"] == "silu" and ret["decay"] == [0.97, 0.8]
    ff = spec.layers[0].feed_forward
    assert (ff.kind, ff["ff"], ff["experts"], ff["top"], ff["groups"], ff["keep"]) == ("routed_experts", 40, 6, 2, 3, 2)
    assert spec.layers[1].feed_forward["groups"] == 1 and spec.layers[3].feed_forward.kind == "none" and spec.layers[4].feed_forward.kind == "none"


@pytest.mark.parametrize("name", sorted(du.CONFIGS))
def test_the_declared_tensors_are_the_checkpoints(name):
    from mimirmind_b200.weights.store import expected_tensors
    _, spec = parse(du.CONFIGS[name])
    assert {k: tuple(v.shape) for k, v in expected_tensors(spec).items()} == du.tensor_shapes(du.CONFIGS[name])


def test_the_rows_of_a_distance_table_may_be_left_to_the_checkpoint():
    from mimirmind_b200.weights.store import expected_tensors
    cfg = copy.deepcopy(du.CONFIGS["P"])
    del cfg["layers"][0]["mixer"]["left"]["bias_rows"]
    _, spec = parse(cfg)
    assert tuple(expected_tensors(spec)["l0.mix.left.rel"].shape) == (-1, 4)
    assert tuple(expected_tensors(spec)["l3.mix.left.rel"].shape) == (8, 2)


@pytest.mark.parametrize("edit,message", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "heads"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("bias_max"), "layers[0].mixer.left.bias_max"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.9]), "decay"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=13), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "layers[1].mixer.conv"),
    (lambda c: c["layers"][1].update(type="lstm"), "lstm"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "dense"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "router"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "router"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_a_wrong_configuration_names_its_key(edit, message):
    from mimirmind_b200.config.model_config import ConfigError
    cfg = copy.deepcopy(du.CONFIGS["P"])
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        parse(cfg)
    assert message in str(e.value)


def test_rows_by_distance():
    from mimirmind_b200.parts.sink_attention import distance_rows
    for rows, far in ((10, 37), (7, 20.5), (32, 300), (2, 1.5), (16, 130)):
        got = distance_rows(rows, far)
        assert len(got) == math.ceil(far) + 1 and got[-1] == rows - 1
        assert got == [pd.distance_bucket(n, rows, far) for n in range(len(got))]
        assert all(b >= a for a, b in zip(got, got[1:])) and got[:rows // 2] == list(range(rows // 2))
        assert all(pd.distance_bucket(n, rows, far) == rows - 1 for n in (len(got), len(got) + 1, 10 * len(got)))
    with pytest.raises(ValueError):
        distance_rows(10, 5)


# ---- the plain mechanisms against hand-made cases --------------------------------------------------------------------
def test_plain_router():
    z = np.log(np.array([[1.0, 2.0, 9.0, 3.0, 4.0, 5.0]]))
    idx, w = pd.route(z, 2, 1, 1)
    assert idx.tolist() == [[2, 5]] and np.allclose(w, [[9 / 14, 5 / 14]])
    # three runs of two: scores 2, 9, 5; the two best runs are the second and third; expert 1 is out though it beats expert 3's neighbour
    idx, w = pd.route(z, 3, 3, 2)
    assert idx.tolist() == [[2, 5, 4]] and np.allclose(w.sum(), 1.0)
    idx, _ = pd.route(z, 2, 3, 1)
    assert idx.tolist() == [[2, 3]]


def test_plain_convolution_and_state_mixers():
    x = np.arange(1.0, 6.0)[:, None]
    taps = np.array([[100.0, 10.0, 1.0]])
    assert pd.causal_conv(x, taps)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    q = np.ones((3, 1, 2))
    k = np.array([[[1.0, 0.0]], [[0.0, 1.0]], [[1.0, 1.0]]])
    v = np.array([[[1.0]], [[10.0]], [[100.0]]])
    o, S = pd.decayed_outer_products(q, k, v, np.array([0.5]))
    assert o[:, 0, 0].tolist() == [1.0, 10.5, 205.25] and S[0, :, 0].tolist() == [100.25, 105.0]
    r = pd.rotate_half(np.array([[[1.0, 5.0, 0.0, 7.0]]]), [1], 2, 1.0)       # pair (0, 1) turned by one radian, the rest passes
    assert np.allclose(r[0, 0], [math.cos(1) - 5 * math.sin(1), 5 * math.cos(1) + math.sin(1), 0.0, 7.0])
    r = pd.rotate_half(np.array([[[1.0, 0.0, 0.0, 0.0]]]), [3], 4, 100.0)     # pairs (0, 2) and (1, 3); the second turns at 1/10 the speed
    assert np.allclose(r[0, 0], [math.cos(3), 0.0, math.sin(3), 0.0])


def test_plain_attention_sink_and_bias():
    q = np.zeros((3, 1, 2))
    k = np.zeros((3, 1, 2))
    v = np.array([[[1.0]], [[2.0]], [[4.0]]])
    rel = np.zeros((4, 1))
    # no scores, no bias, sink logit 0: the sink takes one share of i + 2
    out = pd.biased_sink_attention_core(q, k, v, rel, np.array([0.0]), 1.0, 8)
    assert np.allclose(out[:, 0, 0], [1 / 2, 3 / 3, 7 / 4])
    # a bias on distance 1 of ln 3: that key weighs three times the others
    rel[1, 0] = math.log(3.0)
    out = pd.biased_sink_attention_core(q, k, v, rel, np.array([-1e9]), 1.0, 8)
    assert np.allclose(out[:, 0, 0], [1.0, (3 * 1 + 2) / 4, (1 + 3 * 2 + 4) / 5])
