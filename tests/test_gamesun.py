"""Gamesun without a GPU: its configuration, the description the framework makes of it, the tensors it declares,
what its layers ask of the cache manager, and properties of the plain implementation that the GPU tests lean on."""

import copy

import pytest
import torch

from clockwork_b200.cache import CacheManager
from clockwork_b200.config.registry import architecture_name, shape_config, spec_from_raw
from clockwork_b200.parts import PagedKVNeed, SlotStateNeed, build_model
from clockwork_b200.parts.model import tensor_decls_for_spec
from clockwork_b200.weights.loader import WeightMismatchError, check_declarations
from tests.gamesun_configs import CONFIGS, draw_weights, tensor_shapes
from tests.plain import gamesun_plain as plain


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    config, _, decay_rank = CONFIGS[name]
    spec = spec_from_raw(config)
    assert architecture_name(config) == "Gamesun" and spec.architecture == "Gamesun"
    assert spec.tie_word_embeddings and spec.embedding_scale == config["embedding"]["scale"]
    decls = tensor_decls_for_spec(spec)
    shapes = tensor_shapes(config, decay_rank)
    check_declarations(decls, shapes, "test")  # the decay products' inner size is the checkpoint's; the head is the embedding
    assert {d.name for d in decls if not d.optional} == set(shapes)
    right = {"parallel": "gated_linear", "parallel_2": "decay_linear"}
    for layer, listed in zip(spec.layers, config["layers"]):
        assert (layer.block, layer.mixer.kind) == ("prenorm_residual_short", "side_by_side")
        assert layer.mixer["left"].kind == "window_attention" and layer.mixer["right"].kind == right[listed["type"]]
        assert layer.ffn.kind == ("none" if listed["mlp"] is None else "swiglu")


def test_the_named_shapes_describe_themselves():
    for name in ("gamesun-tiny", "gamesun-2k"):
        spec = spec_from_raw(shape_config(name))
        assert len(tensor_decls_for_spec(spec)) > 10
    assert len(spec_from_raw(shape_config("gamesun-2k", 2)).layers) == 2


def test_a_wrong_shape_and_a_missing_tensor_are_reported():
    config, _, decay_rank = CONFIGS["A"]
    shapes = tensor_shapes(config, decay_rank)
    shapes["l0.mix.left.talk"] = (5, 4)
    del shapes["l1.mix.left.temp"]
    with pytest.raises(WeightMismatchError) as err:
        check_declarations(tensor_decls_for_spec(spec_from_raw(config)), shapes, "test")
    assert err.value.missing == ["l1.mix.left.temp"] and [w[0] for w in err.value.wrong_shape] == ["l0.mix.left.talk"]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="parallel_3"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "unknown feed-forward"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("mask"), "lacks 'size'"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("tau"), "lacks 'tau'"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.9]), "one number per head"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=2), "not a multiple"),
    (lambda c: c.pop("embedding"), "lacks 'scale'"),
    (lambda c: c.update(layers=[]), "non-empty list"),
])
def test_a_faulty_configuration_is_refused(change, message):
    config = copy.deepcopy(CONFIGS["A"][0])
    change(config)
    with pytest.raises(ValueError, match=message):
        build_model(spec_from_raw(config), torch.float32, "cpu")


def test_a_layer_keeps_pages_and_a_state_slot():
    """Rows of [key | value] per key/value head in a windowed page group, and the linear attention's state."""
    config = CONFIGS["A"][0]
    needs = build_model(spec_from_raw(config), torch.float32, "cpu").cache_needs()
    for i, layer in enumerate(config["layers"]):
        left, right = layer["mixer"]["left"], layer["mixer"]["right"]
        assert needs[i] == (PagedKVNeed(left["kv_heads"], left["dim"] + left["vdim"], left["mask"]["size"], planes=1),
                            SlotStateNeed((right["heads"] * right["dim"] * right["vdim"],)))
    cache = CacheManager(needs, num_pages=12, page_size=4, num_state_slots=2)
    assert len(cache.groups) == 4 and sorted(cache.state.needs) == [0, 1, 2, 3]
    req = cache.open("a")
    cache.reserve(req, 30)
    req.num_computed = 30
    assert cache.release_behind_window(req, 30) > 0
    held = {cache.groups[g].need.window: sum(p >= 0 for p in req.tables[g]) for g in range(4)}
    assert held[1] == 1 and held[7] == 2 and held[21] == 6 and held[50] == 8  # pages that a window of that size still reaches
    cache.close("a")
    cache.check_invariants()


def test_two_paged_mixers_side_by_side_are_refused():
    from clockwork_b200.config import PartSpec

    left = PartSpec("window_attention", dict(hidden_size=16, heads=2, kv_heads=1, dim=8, vdim=8, window=4, scale=0.3))
    with pytest.raises(ValueError, match="one layer has one of each"):
        from clockwork_b200.parts import build_part

        build_part("mixer", PartSpec("side_by_side", dict(hidden_size=16, eps=1e-5, left=left, right=left)), "m", torch.float32, "cpu")


def test_the_plain_implementation_does_not_look_ahead_and_forgets_behind_its_windows():
    config, _, decay_rank = CONFIGS["A"]
    w = draw_weights(config, decay_rank, seed=3)
    tokens = list(range(5, 45))
    whole = plain.forward(config, w, tokens, dtype=torch.float64)
    other = tokens[:21] + [t + 1 for t in tokens[21:]]
    assert torch.allclose(plain.forward(config, w, other, dtype=torch.float64)[:21], whole[:21], atol=1e-9)
    # a window of one more or one less token is another function, and so is a state that starts late
    for size in (20, 22):
        changed = copy.deepcopy(config)
        changed["layers"][0]["mixer"]["left"]["mask"]["size"] = size
        assert float((plain.forward(changed, w, tokens, dtype=torch.float64) - whole).abs().max()) > 1e-2
    x = torch.randn(40, config["width"], dtype=torch.float64)
    wd = {k: v.double() for k, v in w.items()}
    for layer, kind in ((0, plain.channel_decay_mixer), (1, plain.head_decay_mixer)):
        m = config["layers"][layer]["mixer"]["right"]
        full = kind(x, wd, f"l{layer}.mix.right", m, 1e-5)
        late = kind(x[25:], wd, f"l{layer}.mix.right", m, 1e-5)
        assert float((full[25:] - late).abs().max()) > 1e-2
