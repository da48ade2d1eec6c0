"""Rapitar without a GPU: its configuration, the description the framework makes of it, and the tensors it declares."""

import copy

import pytest
import torch

from clockwork_b200.config.registry import architecture_name, spec_from_raw
from clockwork_b200.parts.model import tensor_decls_for_spec
from clockwork_b200.weights.loader import WeightMismatchError, check_declarations
from tests.plain import rapitar_plain as plain
from tests.rapitar_configs import CONFIGS, draw_weights, tensor_shapes


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    config, _, decay_rank = CONFIGS[name]
    spec = spec_from_raw(config)
    assert architecture_name(config) == "Rapitar" and spec.architecture == "Rapitar"
    decls = tensor_decls_for_spec(spec)
    shapes = tensor_shapes(config, decay_rank)
    check_declarations(decls, shapes, "test")  # the decay products' inner size is the checkpoint's
    assert {d.name for d in decls} == set(shapes)
    kinds = [(layer.block, layer.mixer.kind, layer.ffn.kind) for layer in spec.layers]
    want = {"dense": "gelu_mlp", "moe": "moe"}
    assert kinds == [("parallel_residual", l["type"], "none" if l["mlp"] is None else want[l["mlp"]["kind"]]) for l in config["layers"]]


def test_a_wrong_shape_and_a_missing_tensor_are_reported():
    config, _, decay_rank = CONFIGS["A"]
    shapes = tensor_shapes(config, decay_rank)
    shapes["l1.mix.in"] = (shapes["l1.mix.in"][0] + 1, shapes["l1.mix.in"][1])
    del shapes["l0.mix.sink"]
    with pytest.raises(WeightMismatchError) as err:
        check_declarations(tensor_decls_for_spec(spec_from_raw(config)), shapes, "test")
    assert err.value.missing == ["l0.mix.sink"] and [w[0] for w in err.value.wrong_shape] == ["l1.mix.in"]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown feed-forward"),
    (lambda c: c["layers"][1]["mixer"].pop("state"), "lacks 'state'"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=4), "rot.dims"),
    (lambda c: c.pop("width"), "lacks 'width'"),
    (lambda c: c.update(layers=[]), "non-empty list"),
])
def test_a_faulty_configuration_is_refused(change, message):
    config = copy.deepcopy(CONFIGS["A"][0])
    change(config)
    with pytest.raises(ValueError, match=message):
        spec_from_raw(config)


def test_cache_needs_by_layer_kind():
    from clockwork_b200.parts import PagedKVNeed, SlotStateNeed, build_model

    config = CONFIGS["C"][0]
    needs = build_model(spec_from_raw(config), torch.float32, "cpu").cache_needs()
    first, last = config["layers"][0]["mixer"], config["layers"][2]["mixer"]
    assert needs[0] == PagedKVNeed(1, first["kv_rank"] + first["rot_dim"], None, planes=1)
    assert needs[2] == PagedKVNeed(1, last["kv_rank"] + last["rot_dim"], None, planes=1)
    wkv = config["layers"][1]["mixer"]
    assert needs[1] == SlotStateNeed((wkv["heads"] * wkv["dim"] ** 2 + config["width"],))
    config = CONFIGS["B"][0]
    needs = build_model(spec_from_raw(config), torch.float32, "cpu").cache_needs()
    m = config["layers"][1]["mixer"]
    channels = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
    assert needs[1] == SlotStateNeed((m["heads"] * m["state"] * m["vdim"] + (m["conv"] - 1) * channels,))
    assert all(isinstance(n, SlotStateNeed) for n in needs.values())


def test_the_plain_implementation_does_not_look_ahead():
    """A token's logits depend on the tokens before it only (every mixer is causal)."""
    config, _, decay_rank = CONFIGS["A"]
    w = draw_weights(config, decay_rank, seed=3)
    tokens = list(range(5, 25))
    whole = plain.forward(config, w, tokens, dtype=torch.float64)
    assert torch.allclose(plain.forward(config, w, tokens[:11], dtype=torch.float64), whole[:11], atol=1e-9)
    other = tokens[:11] + [t + 1 for t in tokens[11:]]
    assert torch.allclose(plain.forward(config, w, other, dtype=torch.float64)[:11], whole[:11], atol=1e-9)
