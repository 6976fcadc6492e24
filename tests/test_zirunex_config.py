"""Zirunex without a GPU: configuration, weight checks, random model folders, the cache manager's kept first
pages, and the plain implementation's own mask and softmax."""

from __future__ import annotations

import copy
import json
import math

import pytest
import torch

from research_2_b200 import models  # noqa: F401  (registers the architectures)
from research_2_b200.cache import CacheManager, GroupSpec
from research_2_b200.cache.arena import MemberSpec, derive_groups
from research_2_b200.config import ConfigError, ZirunexConfig, architecture_of, load_config
from research_2_b200.models import zirunex
from research_2_b200.weights.loader import WeightError, load_weights
from research_2_b200.weights.safetensors_io import read_file, write_file
from tests.plain import zirunex_plain as plain
from tests.zirunex_cases import CASES, make_model_dir


def test_config_is_read_key_by_key():
    cfg = ZirunexConfig.from_json(CASES["c"]["config"])
    assert (cfg.vocab_size, cfg.width, cfg.norm_eps, cfg.embedding_scale) == (300, 128, 1e-5, 4.0)
    assert [layer.weights_of for layer in cfg.layers] == [None, None, 1, 0]
    first = cfg.layers[0].mixer
    assert (first.heads, first.kv_heads, first.dim, first.vdim, first.window, first.keep_first, first.scale) == (8, 1, 64, 64, 70, 5, 0.125)
    assert cfg.layers[1].mlp.ff == 64 and cfg.layers[1].mlp.limit == 1.0
    assert ZirunexConfig.from_json(cfg.to_json()) == cfg
    assert architecture_of(CASES["a"]["config"]).name == "Zirunex"
    assert ZirunexConfig.from_json(CASES["a"]["config"]).layers[1].mlp is None


@pytest.mark.parametrize("path, value, message", [
    (("vocab",), None, "'vocab' is missing"),
    (("norm", "eps"), -1.0, "must be positive"),
    (("layers", 0, "mixer", "dim"), None, "mixer.'dim' is missing"),
    (("layers", 0, "mixer", "scale"), None, "mixer.'scale' is missing"),
    (("layers", 0, "mixer", "kv_heads"), 3, "not a multiple"),
    (("layers", 0, "type"), "recurrent", "not supported"),
    (("layers", 0, "mlp", "kind"), "routed", "not supported"),
    (("layers", 2, "weights_of"), 2, "must name another layer"),
    (("layers", 2, "mlp", "ff"), 80, "describes another layer"),
])
def test_config_errors_name_the_key(path, value, message):
    data = copy.deepcopy(CASES["a"]["config"])
    at = data
    for key in path[:-1]:
        at = at[key]
    if value is None or value == "absent":
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        ZirunexConfig.from_json(data)


def test_what_a_file_does_not_mention_is_not_there():
    data = copy.deepcopy(CASES["d"]["config"])
    layer = data["layers"][1]
    layer["mixer"] = copy.deepcopy(layer["mixer"])   # (the cases' layers share their mixer entries)
    del layer["mlp"], layer["mixer"]["mask"], layer["mixer"]["kv_heads"], layer["mixer"]["vdim"]
    del data["embedding"]
    del data["layers"][0]["mixer"]["mask"]["keep_first"]
    cfg = ZirunexConfig.from_json(data)
    bare = cfg.layers[1]
    assert bare.mlp is None and bare.mixer.kv_heads == bare.mixer.heads == 4 and bare.mixer.vdim == bare.mixer.dim == 32
    assert bare.mixer.window >= 1 << 30 and bare.mixer.keep_first == 0 and cfg.embedding_scale == 1.0
    assert cfg.layers[0].mixer.window == 33 and cfg.layers[0].mixer.keep_first == 0
    assert ZirunexConfig.from_json(cfg.to_json()) == cfg


def test_weight_spec_and_model_folder(tmp_path):
    folder = make_model_dir(tmp_path / "m", CASES["a"])
    arch, cfg = load_config(folder)
    names = [t.name for t in arch.weight_spec(cfg).tensors]
    assert "l0.mix.q.norm" in names and "l1.mix.g" in names and "head" in names
    assert not any(n.startswith("l2.") for n in names), "a layer that borrows has no tensors"
    assert not any(n.startswith("l1.mlp.") for n in names), "a layer without a feed-forward has none"
    tensors = load_weights(folder, arch.weight_spec(cfg))
    assert tensors["l0.mix.q"].shape == (4 * 16, 64) and tensors["l0.mix.o"].shape == (64, 4 * 16) and tensors["l0.mlp.down"].shape == (64, 96)
    stored = read_file(folder / "model.safetensors")
    del stored["l1.mix.k.norm"]
    stored["l2.norm1"] = torch.zeros(64)
    stored["l0.mlp.up"] = torch.zeros(95, 64)
    write_file(folder / "model.safetensors", stored)
    with pytest.raises(WeightError) as err:
        load_weights(folder, arch.weight_spec(cfg))
    assert err.value.missing == ["l1.mix.k.norm"] and err.value.unexpected == ["l2.norm1"] and "l0.mlp.up" in err.value.wrong[0]


def test_schedule_runs_borrowers_with_their_lenders_parts():
    cfg = ZirunexConfig.from_json(CASES["c"]["config"])
    spec = zirunex.model_spec(cfg)
    assert len(spec.layers) == 2
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (1, 2), (0, 3)]
    assert spec.layers[0].block == "parallel" and spec.layers[0].norm_2 is None and spec.embedding_scale == 4.0
    cfg_a = ZirunexConfig.from_json(CASES["a"]["config"])
    assert zirunex.model_spec(cfg_a).layers[1].feed_forward is None


def test_groups_by_window_and_kept_tokens():
    members = [MemberSpec(2, 16, 24, 16, 3), MemberSpec(2, 32, 17, 32, 0), MemberSpec(2, 16, 24, 16, 3), MemberSpec(1, 8, 0, 8, 9)]
    groups, index = derive_groups(members, 8, 10)
    assert index == [0, 1, 0, 2]
    assert [(g.window, g.keep_first) for g in groups] == [(24, 3), (17, 0), (0, 0)], "without a window nothing needs keeping"


def test_cache_manager_keeps_the_first_pages_of_a_window_group():
    page, window, keep = 4, 10, 6
    cm = CacheManager([GroupSpec(page, window, 24, keep)], 2, 200)
    cm.open(0)
    held = []
    for n in range(1, 121):
        cm.slide(0, n - 1)
        cm.reserve(0, n - 1, n)
        table = cm.table(0)
        pos = n - 1
        for j in range(n):  # every key that the row at `pos` reads has a page; no page is held that no later row reads
            assert (table[j // page] != 0) >= plain.sees(pos, j, window, keep), (pos, j)
        want = {j // page for j in range(n) if any(plain.sees(p, j, window, keep) for p in range(pos, pos + 1000))}
        assert {i for i, pg in enumerate(table) if pg} == want, (n, want)
        held.append(cm.pages_held(0))
        assert cm.check() == ""
    assert max(held) <= 2 + 4 and held[-1] == held[-1 - page]
    assert cm.worst_pages(0, 120, 1, 1) == max(held)
    cm.close(0)
    assert cm.n_free(0) == 24
    # a portion of a prompt needs the window of its first row and its own rows
    cm.open(1)
    cm.reserve(1, 0, 50)
    cm.slide(1, 50)
    cm.reserve(1, 50, 83)
    table = cm.table(1)
    assert [i for i, pg in enumerate(table) if pg] == [0, 1] + list(range((50 - window + 1) // page, -(-83 // page)))


def test_the_plain_mask_and_softmax():
    assert [j for j in range(12) if plain.sees(11, j, 4, 2)] == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(12) if plain.sees(3, j, 4, 2)] == [0, 1, 2, 3]
    assert [j for j in range(3) if plain.sees(1, j, 1, 0)] == [1]
    s = torch.tensor([[0.5, -1.0, 2.0], [-math.inf, 0.0, -math.inf], [-80.0, -90.0, -math.inf]], dtype=torch.float64)
    p = plain.sink_softmax(s)
    assert torch.allclose(p[0], torch.exp(s[0]) / (1 + torch.exp(s[0]).sum()))
    assert torch.allclose(p[1], torch.tensor([0.0, 0.5, 0.0], dtype=torch.float64))
    assert float(p[2].sum()) < 1e-30 and float(p[2].sum()) > 0
    big = plain.sink_softmax(torch.tensor([[800.0, 799.0]], dtype=torch.float64))
    assert torch.isfinite(big).all() and abs(float(big.sum()) - 1.0) < 1e-12


def test_unbounded_models_get_a_default_length():
    from research_2_b200.config import EngineOptions

    opts = EngineOptions(max_requests=2).validated(zirunex.UNBOUNDED_SEQ_LEN)
    assert opts.max_seq_len == 4096 and opts.num_slabs == 2 * 256
    assert EngineOptions(max_requests=2, max_seq_len=100000).validated(zirunex.UNBOUNDED_SEQ_LEN).max_seq_len == 100000
    assert json.loads(json.dumps(ZirunexConfig.from_json(CASES["b"]["config"]).to_json()))["architecture"] == "Zirunex"
