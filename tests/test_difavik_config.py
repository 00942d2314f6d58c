"""The Difavik design's configuration and plan, and the cache manager's kept first pages (CPU)."""

import copy

import pytest
import torch

import difavik_configs as DC
from ninfer_amd_mi50_b200.cache.manager import CacheManager
from ninfer_amd_mi50_b200.config.model_config import ConfigError
from ninfer_amd_mi50_b200.engine.loading import build_model
from ninfer_amd_mi50_b200.parts.base import CacheSpec
from ninfer_amd_mi50_b200.registry import architecture_names


def test_the_design_is_registered():
    assert "Difavik" in architecture_names()


@pytest.mark.parametrize("name", sorted(DC.CONFIGS))
def test_every_layer_has_cache_and_state_of_its_own_and_borrowers_add_no_tensors(name):
    cfg, _ = DC.CONFIGS[name]
    typed, model = build_model(cfg)
    n = len(cfg["layers"])
    assert [c.cache for c in model.order] == list(range(n)) and [c.state_slot() for c in model.order] == list(range(n))
    owners = [i for i, L in enumerate(cfg["layers"]) if L.get("weights_of") is None]
    assert len(model.blocks) == len(owners)
    for i, c in enumerate(model.order):
        assert owners[c.layer] == typed.owner(i)
    names = [s.name for s in model.tensor_specs()]
    assert len(names) == len(set(names))
    for i, L in enumerate(cfg["layers"]):
        has = any(x.startswith(f"l{i}.") for x in names)
        assert has == (L.get("weights_of") is None)
    kinds = [L["type"] for L in cfg["layers"]]
    assert [s is not None for s in model.cache_specs()[:n]] == [k == "parallel" for k in kinds]
    assert all(s is not None for s in model.state_specs()[:n])
    # the pair table keeps the previous token in a state slot after the layers'
    assert len(model.state_specs()) == n + (1 if cfg.get("embedding") else 0)
    assert ("bigram" in names) == bool(cfg.get("embedding"))
    assert "head" not in names and "embed" in names


def test_sizes_and_constants_come_from_the_configuration():
    cfg, _ = DC.CONFIGS["borrowing"]
    typed, model = build_model(cfg)
    mix = model.blocks[0].mixer
    left, right = mix.mixers
    assert (left.heads, left.kv_heads, left.head_dim, left.window, left.keep_first) == (6, 2, 16, 21, 3)
    assert left.scale == 0.3 and left.cache_spec() == CacheSpec("window", 2, 16, 21, keep_first=3)
    assert right.decay_values == (0.9, 0.97, 0.995) and abs(right.key_scale - 0.25) < 1e-12
    assert right.position.rotary_dim == 8 and right.position.theta == 500.0
    slopes = left.slopes(torch.device("cpu"))
    assert torch.allclose(slopes, torch.tensor([2.0 ** (-8.0 * (h + 1) / 6) for h in range(6)]))
    ff = model.blocks[0].feed_forward
    assert ff.activation == (2, 1.5, 1.702) and (ff.num_experts, ff.top_k, ff.norm_topk_prob) == (5, 2, False)
    dense = model.blocks[1].feed_forward
    assert dense.activation == (2, 2.5, 1.702) and dense.has_bias
    light = model.blocks[1].mixer
    assert light.silu_qkv and not light.norm_per_head and light.norm_weight and light.key_scale == 1.0


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=24), "values are the keys"),
    (lambda c: c["layers"][0]["mixer"]["right"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][2].update(weights_of=0), "differs"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "buckets"),
])
def test_a_configuration_that_cannot_run_is_refused(change, message):
    cfg = copy.deepcopy(DC.BORROWING)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        build_model(cfg)


def test_a_window_group_never_gives_back_the_pages_of_the_kept_first_tokens():
    spec = CacheSpec("window", 1, 8, window=10, keep_first=20)       # 20 kept tokens: pages 0 and 1 of 16
    cm = CacheManager([spec], [None], page_size=16, num_pages=12, max_requests=2, max_context=160, allocate=False)
    cm.open("a")
    cm.reserve("a", 150)
    cm.commit("a", 150)
    table = cm.block_table(0, "a")
    # positions from 141 on are still read: pages 8 and 9; pages 0 and 1 hold kept tokens
    assert [p >= 0 for p in table] == [True, True] + [False] * 6 + [True, True]
    assert cm.pages_free() == [12 - 4]
    cm.check()
    cm.close("a")
    assert cm.pages_free() == [12]
    plain = CacheManager([CacheSpec("window", 1, 8, window=10)], [None], page_size=16, num_pages=12, max_requests=2,
                         max_context=160, allocate=False)
    plain.open("a")
    plain.reserve("a", 150)
    plain.commit("a", 150)
    assert [p >= 0 for p in plain.block_table(0, "a")] == [False] * 8 + [True, True]
