"""Kagorax on the host: configuration, plan, tensor names, the distance table's rows and the
cache manager's handling of kept first tokens (no GPU)."""
import copy

import pytest

import plain_kagorax as plain
from kagorax_util import ROWS_A, SMALL_A, SMALL_B, random_weights
from tinyinfer_b200.cache import CacheManager
from tinyinfer_b200.cache.manager import RELEASED
from tinyinfer_b200.config import ConfigError, architecture_of
from tinyinfer_b200.parts.base import PagedKVSpec
from tinyinfer_b200.parts.gated_attention import distance_rows
from tinyinfer_b200.parts.model import CausalLM
from tinyinfer_b200.weights.loader import WeightsError, check_tensors


def _plan(cfg):
    arch = architecture_of(cfg)
    return arch.build_plan(arch.from_dict(cfg))


def test_the_architecture_is_chosen_by_its_name():
    assert architecture_of(SMALL_A).name == "Kagorax"
    assert architecture_of({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError):
        architecture_of({"architecture": "Nobody"})


def test_plan_shares_cache_slots_and_keeps_what_the_widest_reader_needs():
    plan = _plan(SMALL_A)
    assert [(e.layer, e.cache_slot, e.writes_cache) for e in plan.schedule] == [(0, 0, True), (1, 0, False), (2, 1, True)]
    specs = CausalLM(plan).cache_specs()
    # layer 1 reads layer 0's slot with a window of 33 and 5 kept tokens: the slot keeps that much
    assert specs[0] == PagedKVSpec(2, 16, 33, 24, 5)
    assert specs[1] == PagedKVSpec(1, 32, 9, None, 0)
    assert plan.layers[1].ffn is None and plan.layers[0].ffn is not None


def test_tensor_names_and_shapes():
    model = CausalLM(_plan(SMALL_A))
    want = model.expected_tensors()
    have = {k: tuple(v.shape) for k, v in random_weights(SMALL_A, ROWS_A, 0).items()}
    assert set(want) == set(have)
    check_tensors("here", want, have)
    assert want["l0.mix.rel"].shape == (None, 4)            # the stored table decides its rows
    assert "l1.mix.k" not in want and "l1.mlp.router" not in want and "l2.mlp.shared.sg" not in want
    wrong = dict(have)
    wrong["l0.mix.rel"] = (8, 5)
    with pytest.raises(WeightsError):
        check_tensors("here", want, wrong)


@pytest.mark.parametrize("change, text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0].__setitem__("type", "recurrent"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "mixer.vdim"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("keep_first"), "mixer.mask.keep_first"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 4), "differ"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "kind"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_bad_configurations_are_refused(change, text):
    cfg = copy.deepcopy(SMALL_A)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        architecture_of(cfg).from_dict(cfg)


@pytest.mark.parametrize("rows, far", [(8, 40), (12, 64), (6, 100), (4, 16), (32, 1024), (16, 128), (7, 50)])
def test_rows_of_the_distance_table(rows, far):
    got = distance_rows(rows, far)
    assert got == [plain.distance_bucket(n, rows, far) for n in range(far + 1)]
    assert got[-1] == rows - 1 and got[: rows // 2] == list(range(rows // 2))
    assert all(a <= b for a, b in zip(got, got[1:]))
    assert plain.distance_bucket(far + 1000, rows, far) == rows - 1


def test_pages_of_the_kept_first_tokens_outlive_the_window():
    page = 4
    cm = CacheManager([PagedKVSpec(1, 8, window=6, keep_first=5)], page_size=page, num_pages=9, max_requests=2)
    cm.reserve_step([("a", 3)])
    cm.release_passed("a")
    for _ in range(10):                       # token by token to 23 tokens
        cm.reserve_step([("a", 2)])
        cm.release_passed("a")
        cm.check()
    table = cm.block_table(0, "a")
    # 5 kept tokens live on blocks 0 and 1; the next token (position 23) reads from 18: block 4 on
    assert table[0] != RELEASED and table[1] != RELEASED
    assert table[2] == RELEASED and table[3] == RELEASED and table[4] != RELEASED
    free_before = cm.free_pages()[0]
    cm.reserve_step([("b", 8)])               # a freed page is used again by another request
    assert cm.free_pages()[0] == free_before - 2
    cm.free_request("a")
    cm.free_request("b")
    cm.check()
    assert cm.free_pages() == [9]


def test_no_kept_tokens_release_as_before():
    cm = CacheManager([PagedKVSpec(1, 8, window=4)], page_size=4, num_pages=6, max_requests=1)
    cm.reserve_step([("a", 13)])
    cm.release_passed("a")
    assert cm.block_table(0, "a")[:2] == [RELEASED, RELEASED]


def test_the_plain_router_prefers_the_lower_index_on_a_tie():
    import torch
    cfg = copy.deepcopy(SMALL_B)
    w = {k: v.double() for k, v in random_weights(cfg, [4, 6], 1).items()}
    w["l0.mlp.router"][1] = w["l0.mlp.router"][0]
    mlp = dict(cfg["layers"][0]["mlp"], router={"experts": 2, "top": 1})
    h = torch.randn((3, 32), dtype=torch.float64)
    only_first = dict(w)
    only_first["l0.mlp.e1.down"] = torch.zeros_like(w["l0.mlp.e1.down"])
    assert torch.equal(plain.routed_experts(h, w, "l0.mlp.", mlp), plain.routed_experts(h, only_first, "l0.mlp.", mlp))
