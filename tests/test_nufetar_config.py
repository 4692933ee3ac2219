"""Nufetar on the CPU: the configuration reader, the parts it picks, tensor names, caches, and the cache
manager's handling of runs of positions (chunks) and of caches without a value pool."""
import copy

import pytest
import torch

from mlx_lm_b200.cache import CacheManager
from mlx_lm_b200.config import ConfigError, get_architecture
from mlx_lm_b200.parts import (LatentAttention, LearnedActMLP, PagedKVSpec, StateSpec, TalkingHeadsAttention, WKVMixer)
from mlx_lm_b200.weights.loader import random_tensors
from nufetar_cases import CONFIG_A, CONFIG_B, CONFIG_C


def describe(config, shapes=None):
    arch = get_architecture(config)
    args = arch.args_class.from_dict(copy.deepcopy(config))
    if shapes is not None:
        args.sizes_from_tensors(shapes)
    return arch.build(args)


def test_found_by_its_architecture_key_and_parts_follow_the_layer_list():
    d = describe(CONFIG_A)
    assert d.model_type == "nufetar"
    kinds = [type(b.mixer) for b in d.blocks]
    assert kinds == [TalkingHeadsAttention, LatentAttention, WKVMixer, TalkingHeadsAttention]
    assert [isinstance(b.feed_forward, LearnedActMLP) for b in d.blocks] == [True, True, False, True]
    assert d.head.tied_to is d.embedding
    a, l = d.blocks[0].mixer, d.blocks[1].mixer
    assert (a.chunk, a.window, a.interleaved, a.scale) == (24, None, False, 0.2)
    assert (l.window, l.chunk, l.interleaved) == (20, None, True)
    assert d.blocks[3].mixer.chunk == 50


def test_tensor_names_and_shapes():
    d = describe(CONFIG_B)
    specs = {s.name: tuple(s.shape) for s in d.param_specs()}
    D = 96
    assert specs["embed"] == (200, D) and specs["final.norm"] == (D,)
    assert specs["l0.mix.mu.w"] == (D,) and specs["l0.mix.w1"] == (5, D) and specs["l0.mix.w2"] == (144, 5)
    assert specs["l0.mix.w0"] == (144,) and specs["l0.mix.u"] == (3, 48) and specs["l0.mix.norm"] == (144,)
    assert specs["l0.mix.r"] == specs["l0.mix.g"] == (144, D) and specs["l0.mix.o"] == (D, 144)
    assert specs["l0.mlp.up"] == (256, D) and specs["l0.mlp.down"] == (D, 256) and specs["l0.mlp.act"] == (2,)
    assert specs["l1.mix.q"] == (40, D) and specs["l1.mix.dkv"] == (56, D) and specs["l1.mix.dkv.norm"] == (40,)
    assert specs["l1.mix.uk"] == (24, 40) and specs["l1.mix.uv"] == (40, 40) and specs["l1.mix.o"] == (D, 40)
    assert "l1.mlp.up" not in specs and "l1.norm2" not in specs
    assert specs["l2.mix.q"] == (144, D) and specs["l2.mix.k.b"] == (144,) and specs["l2.mix.v"] == (120, D)
    assert specs["l2.mix.talk"] == (3, 3) and specs["l2.mix.g"] == (3, D) and specs["l2.mix.o.b"] == (D,)
    assert "l2.mix.g.b" not in specs
    assert len(set(specs)) == len(d.param_specs())


def test_caches():
    specs = describe(CONFIG_C).cache_specs()
    assert specs[0] == PagedKVSpec(1, 16, None, chunk=7, value_dim=24)
    assert specs[(1, "shift")] == StateSpec((80,)) and specs[(1, "wkv")] == StateSpec((5, 16, 16))
    assert specs[2] == PagedKVSpec(1, 40, 300, value_dim=0)         # a row of 30 + 6, stored 40 wide; no value pool
    assert specs[3] == PagedKVSpec(2, 64, None, chunk=64, value_dim=8)


def test_the_decay_rank_comes_from_a_tensor_where_the_configuration_is_silent():
    config = copy.deepcopy(CONFIG_A)
    del config["layers"][2]["mixer"]["decay_rank"]
    assert describe(config, {"l2.mix.w1": (11, 64)}).blocks[2].mixer.decay_rank == 11
    assert describe(config).blocks[2].mixer.decay_rank == 32
    assert describe(CONFIG_A, {"l2.mix.w1": (11, 64)}).blocks[2].mixer.decay_rank == 8      # a key wins


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 4), "rot_dim"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "experts"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][2]["mixer"].pop("heads"), "heads"),
])
def test_a_wrong_configuration_is_named(edit, word):
    config = copy.deepcopy(CONFIG_A)
    edit(config)
    with pytest.raises(ConfigError, match=word):
        describe(config)


def test_random_weights_are_the_same_for_the_same_seed():
    d = describe(CONFIG_A)
    a, b = random_tensors(d, 3), random_tensors(d, 3)
    assert all(torch.equal(a[k], b[k]) for k in a) and set(a) == {s.name for s in d.param_specs()}


def test_pages_before_the_current_run_are_given_back():
    """A cache whose positions read only their own run of ``chunk`` positions: once a request has moved into a new
    run, the pages that lie wholly before it return to the pool; the page in which the run starts stays."""
    mgr = CacheManager({0: PagedKVSpec(1, 16, None, chunk=40)}, page_size=16, n_pages=8, max_len=512)
    mgr.add_request("a")
    mgr.reserve("a", 39)
    mgr.commit("a")
    assert mgr.pages_in_use() == [3]
    mgr.reserve("a", 1)          # position 39, the last of the first run
    mgr.commit("a")              # the next position, 40, starts a run: pages 0 and 1 go, the page of 32..47 stays
    assert mgr.pages_in_use() == [1] and mgr.requests["a"].pages[0][:3] == [-1, -1, mgr.requests["a"].pages[0][2]]
    mgr.reserve("a", 100)        # positions 40..139: runs start at 80 and 120
    mgr.commit("a")
    assert mgr.requests["a"].pages[0][:7] == [-1] * 7 and mgr.pages_in_use() == [2]     # 120 // 16 = 7
    mgr.check()
    mgr.release("a")
    assert mgr.pages_in_use() == [0]


def test_a_window_and_runs_together_keep_what_both_need():
    mgr = CacheManager({0: PagedKVSpec(1, 16, 20, chunk=64)}, page_size=16, n_pages=8, max_len=512)
    mgr.add_request("a")
    mgr.reserve("a", 70)
    mgr.commit("a")              # next position 70: the window starts at 51, the run at 64: page 4 on
    assert mgr.requests["a"].pages[0][:5] == [-1, -1, -1, -1, mgr.requests["a"].pages[0][4]]
