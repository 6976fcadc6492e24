"""Bosenex without a GPU: configuration keys and their errors, the tensors a checkpoint must hold, the parts that a
configuration becomes, and the cache and state members that they ask for."""

from __future__ import annotations

import copy

import pytest
import torch

from research_2_b200 import models  # noqa: F401  (registers the architectures)
from research_2_b200.config.bosenex import BosenexConfig, ExpertsMlp, MatrixMemoryMixer, SideBySideMixer
from research_2_b200.config.registry import ConfigError, architecture_of
from research_2_b200.models.bosenex import model_spec, random_weights, weight_spec
from research_2_b200.weights.loader import WeightError, check_and_select
from tests.bosenex_cases import CASES


def test_every_case_parses_and_round_trips():
    for name, case in CASES.items():
        arch = architecture_of(case["config"])
        cfg = arch.parse_config(case["config"])
        assert arch.name == "Bosenex" and isinstance(cfg, BosenexConfig)
        again = arch.parse_config(arch.config_to_json(cfg))
        assert again == cfg, name


def test_what_a_file_does_not_mention_is_not_there():
    cfg = BosenexConfig.from_json(CASES["b"]["config"])
    assert cfg.embedding_scale == 1.0 and cfg.logit_scale == 1.0
    left = cfg.layers[1].mixer.left
    assert left.rot_dims == 0 and left.window == 1 and left.softcap == 5.0
    assert cfg.layers[0].mixer.left.softcap == 0.0
    assert isinstance(cfg.layers[0].mlp, ExpertsMlp) and cfg.layers[0].mlp.shared_ff == 0
    cfg = BosenexConfig.from_json(CASES["c"]["config"])
    assert isinstance(cfg.layers[0].mixer, MatrixMemoryMixer) and cfg.layers[0].mixer.gate_cap == 0.0
    cfg = BosenexConfig.from_json(CASES["d"]["config"])
    assert isinstance(cfg.layers[0].mixer, SideBySideMixer) and cfg.layers[0].mixer.left.window == 0 and cfg.layers[0].mlp is None
    minimal = {"heads": 2, "dim": 8, "scale": 0.5}
    data = copy.deepcopy(CASES["b"]["config"])
    data["layers"][0]["mixer"]["left"] = minimal
    data["layers"][0]["mixer"]["right"] = {"heads": 2, "vdim": 4, "state": 3, "conv": 2}
    cfg = BosenexConfig.from_json(data)
    m = cfg.layers[0].mixer
    assert (m.left.kv_heads, m.left.vdim, m.left.window, m.right.groups, m.right.norm_groups) == (2, 8, 0, 1, 1)


@pytest.mark.parametrize("path, value, text", [
    (("vocab",), None, "'vocab'"), (("width",), 0, "'width'"), (("norm", "eps"), None, "norm.'eps'"),
    (("layers", 0, "type"), "conv", "'type'"), (("layers", 0, "mixer", "left", "heads"), None, "left.'heads'"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "multiple"), (("layers", 0, "mixer", "left", "rot", "dims"), 7, "even"),
    (("layers", 0, "mixer", "right", "state"), None, "right.'state'"), (("layers", 0, "mixer", "right", "groups"), 3, "multiple"),
    (("layers", 1, "mixer", "dim"), "x", "'dim'"), (("layers", 1, "mlp", "router", "top"), 9, "'top'"),
    (("layers", 1, "mlp", "kind"), "sparse", "'kind'"), (("layers", 0, "mlp", "ff"), None, "mlp.'ff'"),
    (("layers", 1, "mlp", "expert", "limit"), -1.0, "'limit'"),
])
def test_errors_name_the_key(path, value, text):
    data = copy.deepcopy(CASES["a"]["config"])
    at = data
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError) as err:
        BosenexConfig.from_json(data)
    assert text in str(err.value), str(err.value)


def test_weight_spec_and_loader_errors():
    cfg = BosenexConfig.from_json(CASES["a"]["config"])
    spec = weight_spec(cfg)
    names = {t.name: t.shape for t in spec.tensors}
    assert names["l0.mix.left.q"] == (64, 64) and names["l0.mix.left.g"] == (4, 64) and names["l0.mix.left.sink"] == (4,)
    assert names["l0.mix.right.in"] == (2 * 32 + 2 * 8 + 2, 64) and names["l0.mix.right.conv"] == (48, 4)
    assert names["l1.mix.i"] == (2, 64) and names["l1.mix.f.b"] == (2,) and names["l1.mix.norm"] == (32,)
    assert names["l1.mlp.e3.down"] == (64, 32) and names["l1.mlp.shared.gate"] == (48, 64) and names["l1.mlp.router.b"] == (4,)
    assert "l2.norm2" not in names and not any(n.startswith("l2.mlp.") for n in names), "a layer without a feed-forward"
    assert "l3.mlp.shared.up" not in names and names["l0.mlp.up"] == (96, 64)
    weights = random_weights(cfg, 0)
    assert set(weights) == set(names) and all(tuple(weights[n].shape) == s for n, s in names.items())
    assert check_and_select(dict(weights), spec).keys() == names.keys()
    broken = dict(weights)
    del broken["l1.mix.f.b"]
    broken["l0.mix.left.sink"] = torch.zeros(5)
    broken["l9.extra"] = torch.zeros(1)
    with pytest.raises(WeightError) as err:
        check_and_select(broken, spec)
    assert err.value.missing == ["l1.mix.f.b"] and err.value.unexpected == ["l9.extra"] and "l0.mix.left.sink" in err.value.wrong[0]


def test_parts_and_members():
    from research_2_b200.cache.arena import derive_groups

    cfg = BosenexConfig.from_json(CASES["a"]["config"])
    spec = model_spec(cfg)
    assert [layer.mixer.kind for layer in spec.layers] == ["side_by_side", "mlstm", "mlstm", "side_by_side"]
    assert [None if layer.feed_forward is None else layer.feed_forward.kind for layer in spec.layers] == ["gated_mlp", "routed_experts", None, "routed_experts"]
    assert spec.layers[2].norm_2 is None and spec.layers[0].block == "pre_norm"
    assert spec.final_norm.params["gain_scale"] == 0.5 and spec.embedding_scale == 4.0
    left = spec.layers[3].mixer.params["left"]
    assert left["kind"] == "rotary_window_attention" and left["params"]["window"] == 7 and left["params"]["rot_dims"] == 8
    assert spec.layers[3].feed_forward.params["shared_limit"] is None and spec.layers[1].feed_forward.params["shared_limit"] == 2.0
    # windows of 24 and 7 tokens: two cache groups, each giving pages back as its window passes
    from research_2_b200.cache.arena import MemberSpec
    groups, index = derive_groups([MemberSpec(2, 16, 24, 16, 0), MemberSpec(2, 32, 7, 8, 0)], 16, 10)
    assert [g.window for g in groups] == [24, 7] and index == [0, 1]
