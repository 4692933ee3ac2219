"""Lelatar without a GPU: configuration, tensor names, the run order of a looped span with a cache per pass,
blocks with several named caches in the cache manager, and the plain implementation against itself."""
import copy

import pytest
import torch

import plain_lelatar as plain
from lelatar_cases import CONFIG_P, CONFIG_Q, CONFIG_R, CONFIG_S, CONFIG_T, ONLY_MAMBA, tokens
from mlx_lm_b200.cache import CacheManager
from mlx_lm_b200.config import ConfigError, get_architecture
from mlx_lm_b200.parts import PagedKVSpec, Reentry, RunEntry, StateSpec
from mlx_lm_b200.weights.loader import random_tensors


def describe(config):
    arch = get_architecture(config)
    return arch.build(arch.args_class.from_dict(copy.deepcopy(config)))


def test_the_architecture_is_found_by_its_name():
    assert get_architecture({"architecture": "Lelatar"}).model_type == "lelatar"
    assert get_architecture({"model_type": "lelatar"}).model_type == "lelatar"
    with pytest.raises(ConfigError):
        get_architecture({"architecture": "NoSuchDesign"})


def test_tensor_names_and_shapes_follow_the_config():
    d = describe(CONFIG_P)
    specs = {s.name: s.shape for s in d.param_specs()}
    assert specs["embed"] == (96, 64) and specs["head"] == (96, 64) and specs["final.norm"] == (64,)
    assert specs["loop.in"] == (64, 128) and specs["loop.step"] == (2, 64) and specs["side.embed"] == (96, 16)
    assert specs["l0.mix.left.q"] == (4 * 32, 64) and specs["l0.mix.left.k"] == (2 * 32, 64)
    assert specs["l0.mix.left.v"] == (2 * 16, 64) and specs["l0.mix.left.o"] == (64, 4 * 16)
    assert specs["l0.mix.left.q.norm"] == (128,) and specs["l0.mix.left.sink"] == (4,)
    assert specs["l0.mix.right.q.conv"] == (4 * 16, 3) and specs["l0.mix.right.v"] == (4 * 24, 64)
    assert specs["l0.mix.right.norm"] == (24,) and specs["l0.mix.right.b"] == (4, 64)
    assert specs["l0.mlp.gate"] == (80, 64) and specs["l0.mlp.down"] == (64, 80) and "l1.mlp.gate" not in specs
    assert specs["l1.mix.in"] == (2 * 64 + 2 * 16 + 4, 64) and specs["l1.mix.conv"] == (64 + 32, 4)
    assert specs["l1.side.gate"] == (8, 64) and specs["l1.side.proj"] == (64, 8) and "l1.norm2" not in specs
    assert "side.embed" not in {s.name for s in describe(CONFIG_Q).param_specs()}
    assert "loop.in" not in {s.name for s in describe(CONFIG_R).param_specs()}


def test_bad_configurations_are_refused_in_words():
    bad = copy.deepcopy(CONFIG_P)
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ConfigError, match="layers\\[0\\].type"):
        describe(bad)
    bad = copy.deepcopy(CONFIG_P)
    del bad["layers"][1]["mixer"]["state"]
    with pytest.raises(ConfigError, match="state"):
        describe(bad)
    bad = copy.deepcopy(CONFIG_P)
    bad["loop"]["stop"] = 5
    with pytest.raises(ConfigError, match="loop"):
        describe(bad)
    bad = copy.deepcopy(CONFIG_P)
    bad["layers"][0]["mlp"]["kind"] = "experts"
    with pytest.raises(ConfigError, match="kind"):
        describe(bad)


def test_a_looped_span_runs_again_with_caches_of_its_own():
    d = describe(CONFIG_Q)        # 4 layers, layers 1..2 three times
    runs = [(e.block, e.cache_id) if isinstance(e, RunEntry) else ("in", e.index) for e in d.order]
    assert runs == [(0, 0), ("in", 0), (1, 1), (2, 2), ("in", 1), (1, 4), (2, 5), ("in", 2), (1, 6), (2, 7), (3, 3)]
    assert [(i, t, first) for i, t, first in plain.run_order(CONFIG_Q)] == \
        [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (1, 2, True), (2, 2, False),
         (3, None, False)]
    specs = d.cache_specs()
    assert {k[0] for k in specs} == {0, 1, 2, 3, 4, 5, 6, 7}
    assert specs[(2, "left")] == specs[(5, "left")] == PagedKVSpec(1, 64, None)
    assert specs[(7, "right.rule")] == StateSpec((2, 48, 32)) and specs[(4, "conv")] == StateSpec((2, 4 * 24 + 2 * 4 * 8))
    assert sum(isinstance(e, Reentry) for e in describe(CONFIG_R).order) == 0


def test_blocks_with_several_named_caches_in_the_manager():
    d = describe(CONFIG_P)
    mgr = CacheManager(d.cache_specs(), page_size=16, n_pages=6, max_requests=2, max_len=64)
    assert len(mgr.kv_groups) == 1 and mgr.kv_groups[0].cache_ids == [(0, "left"), (2, "left")]
    assert sorted(mgr.names_of(0)) == ["left", "right.conv", "right.rule"] and mgr.names_of(1) == ["conv", "ssm"]
    mgr.add_request("a")
    mgr.reserve("a", 40)
    mgr.commit("a")
    assert mgr.pages_in_use() == [3]
    mgr.add_request("b")
    with pytest.raises(Exception):
        mgr.add_request("c")
    mgr.release("a")
    mgr.add_request("c")          # a's slot, given back
    assert mgr.requests["c"].slot == 0 and mgr.pages_in_use() == [0]
    mgr.check()


@pytest.mark.parametrize("config", [CONFIG_P, CONFIG_Q, CONFIG_R, CONFIG_S, CONFIG_T, ONLY_MAMBA])
def test_the_plain_model_is_causal(config):
    """Logits at a position do not change when tokens are appended (the plain implementation against itself)."""
    w = random_tensors(describe(config), seed=3)
    toks = tokens(30, config["vocab"], 1)
    full = plain.forward(config, w, toks)
    part = plain.forward(config, w, toks[:19])
    assert float((full[:19] - part).abs().max()) < 1e-9
    assert full.shape == (30, config["vocab"]) and bool(torch.isfinite(full).all())
