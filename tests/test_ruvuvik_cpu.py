"""Ruvuvik without a GPU: configuration errors, the plan (layers that run another layer's tensors
on a cache slot of their own), tensor names, what each mixer keeps per request, pages of earlier
chunks going back to the pool, and the plain implementation against itself (a sequence in pieces)."""
import copy

import pytest
import torch

import plain_ruvuvik as plain
from ruvuvik_util import SMALL, SMALL_A, random_weights
from tinyinfer_b200.cache import CacheManager
from tinyinfer_b200.config.registry import ConfigError, architecture_of
from tinyinfer_b200.parts.base import FixedStateSpec, PagedKVSpec
from tinyinfer_b200.parts.model import CausalLM
from util import random_tokens


def _plan(cfg):
    arch = architecture_of(cfg)
    return arch.build_plan(arch.from_dict(cfg))


def test_registry_names_the_design():
    assert architecture_of({"architecture": "Ruvuvik"}).name == "Ruvuvik"


@pytest.mark.parametrize("path,value,text", [
    (("layers", 0, "type"), "conv", "known:"),
    (("layers", 2, "mixer", "kv_heads"), 3, "kv heads"),
    (("layers", 2, "mixer", "rot", "dims"), 5, "even"),
    (("layers", 2, "mixer", "rot", "dims"), 14, "at most"),
    (("layers", 0, "mixer", "rot", "dims"), 2, "rotated part"),
    (("layers", 0, "mlp", "kind"), "moe", "known:"),
    (("layers", 3, "weights_of"), 3, "another layer"),
    (("layers", 3, "weights_of"), 4, "no tensors of its own"),
    (("layers", 3, "weights_of"), 0, "differ"),
    (("layers", 2, "mixer", "scale"), None, "lacks"),
    (("layers", 2, "mixer", "softcap"), -1.0, "positive"),
    (("norm", "eps"), 0, "positive"),
])
def test_configuration_errors(path, value, text):
    cfg = copy.deepcopy(SMALL_A)
    node = cfg
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    with pytest.raises(ConfigError, match=text):
        _plan(cfg)


def test_plan_shares_tensors_and_not_caches():
    plan = _plan(SMALL_A)
    assert len(plan.layers) == 3 and [e.layer for e in plan.schedule] == [0, 1, 2, 1, 2, 0]
    assert [e.cache_slot for e in plan.schedule] == list(range(6)) and all(e.writes_cache for e in plan.schedule)
    model = CausalLM(plan)
    assert set(model.expected_tensors()) == set(random_weights(SMALL_A, 5, 0))
    specs = model.cache_specs()
    assert specs[0] == specs[5] == PagedKVSpec(1, 24, None, 0)
    assert specs[2] == specs[4] == PagedKVSpec(2, 12, None, 8, 0, 7)
    assert specs[1] == specs[3] == FixedStateSpec((2 * 12 * 12 + 48,), torch.float32)
    assert plan.layers[1].ffn is None and plan.layers[1].ffn_norm is None


def test_a_cap_or_a_mask_that_is_not_named_does_not_exist():
    cfg = copy.deepcopy(SMALL_A)
    for i in (2, 4):                      # (the two layers may share one dictionary)
        cfg["layers"][i]["mixer"].pop("softcap", None)
        cfg["layers"][i]["mixer"].pop("mask", None)
    spec = _plan(cfg).layers[2].mixer
    assert spec.params["softcap"] is None and spec.params["chunk"] is None
    assert CausalLM(_plan(cfg)).cache_specs()[2] == PagedKVSpec(2, 12, None, 8, 0, None)


def test_the_decay_width_is_the_stored_tensors():
    model = CausalLM(_plan(SMALL_A))
    assert model.expected_tensors()["l1.mix.w1"].shape == (None, 48)
    cfg = copy.deepcopy(SMALL_A)
    cfg["layers"][1]["mixer"]["decay_rank"] = 9
    cfg["layers"][3]["mixer"]["decay_rank"] = 9
    assert CausalLM(_plan(cfg)).expected_tensors()["l1.mix.w2"].shape == (24, 9)


def test_pages_of_earlier_chunks_go_back():
    cm = CacheManager([PagedKVSpec(2, 8, None, None, 0, 20), PagedKVSpec(1, 12, None, 0)],
                      page_size=8, num_pages=12, max_requests=2)
    cm.reserve_step([("a", 19)])
    assert cm.release_passed("a") == 0                        # position 19 still reads from 0
    cm.reserve_step([("a", 1)])                               # the next token, 20, opens a chunk
    assert cm.release_passed("a") == 2                        # pages 0..7 and 8..15; 16..23 straddles
    assert cm.block_table(0, "a")[:3] == [-1, -1, cm.block_table(0, "a")[2]]
    assert all(p >= 0 for p in cm.block_table(1, "a"))        # the group without chunks keeps everything
    cm.reserve_step([("a", 45)])                              # through chunks 1, 2 into 3 (60..)
    cm.release_passed("a")
    assert [p >= 0 for p in cm.block_table(0, "a")] == [False] * 7 + [True, True]
    cm.check()
    cm.free_request("a")
    assert cm.free_pages() == [12, 12]


def test_plain_implementation_in_pieces_equals_whole():
    cfg, rank = SMALL["A"]
    w = random_weights(cfg, rank, 1)
    tokens = random_tokens(cfg["vocab"], 40, seed=2)
    whole, _ = plain.forward(cfg, w, tokens)
    carry, parts = None, []
    for lo, hi in ((0, 1), (1, 9), (9, 11), (11, 30), (30, 40)):
        out, carry = plain.forward(cfg, w, tokens[lo:hi], carry=carry)
        parts.append(out)
    assert (torch.cat(parts) - whole).abs().max() < 1e-9


def test_plain_mechanisms_at_their_edges():
    # a key outside the chunk has no say; the sink takes its share; the cap bounds the score
    q = torch.zeros((1, 1, 4), dtype=torch.float64)
    q[0, 0, 0] = 1.0
    keys = torch.zeros((6, 1, 4), dtype=torch.float64)
    values = torch.arange(6, dtype=torch.float64).view(6, 1, 1)
    keys[2, 0, 0] = 50.0                                       # the last key of chunk 0
    out = plain.attend(q, keys, values, [5], 1.0, chunk=3)
    assert abs(out.item() - 4.0) < 1e-12                       # mean of values 3, 4, 5
    out = plain.attend(q, keys, values, [2], 1.0, chunk=3)
    assert abs(out.item() - 2.0) < 1e-12                       # inside its chunk it takes everything
    out = plain.attend(q, keys, values, [2], 1.0, chunk=3, cap=1.0)
    e = torch.exp(torch.tensor(1.0, dtype=torch.float64))
    assert abs(out.item() - (0 + 1 + 2 * e) / (2 + e)) < 1e-9  # tanh(50) = 1: the score is capped at 1
    out = plain.attend(q, keys[:1], values[:1] + 1.0, [0], 1.0, sink=torch.tensor([0.0]))
    assert abs(out.item() - 0.5) < 1e-12                       # one key with score 0 against a sink of 0
    z = torch.tensor([-2.0, 0.0, 3.0], dtype=torch.float64)
    y = plain.xielu(z, 0.0, 0.0)
    ln2 = torch.log(torch.tensor(2.0, dtype=torch.float64))
    assert torch.allclose(y, torch.stack([(0.5 + ln2) * (torch.exp(z[0]) - 1 + 2) - 1, z[1], ln2 * 9 + 1.5]))
