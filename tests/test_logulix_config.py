"""Logulix without a GPU: configuration, registry, tensor names, cache specs, random folders."""

import copy
import json

import pytest
import torch

import plain_logulix as PL
import tiny_logulix as L
from mini_llm_stack_b200.cache.manager import CacheManager
from mini_llm_stack_b200.config import build_model, config_from_dict, config_from_folder
from mini_llm_stack_b200.config.model_config import ConfigError
from mini_llm_stack_b200.parts.base import FixedState, PagedKV, PagedWithState
from mini_llm_stack_b200.weights import write_random_model
from mini_llm_stack_b200.weights.loader import open_weights


def test_config_round_trip_and_layer_runs():
    cfg = config_from_dict(L.L_MIXED)
    assert cfg.architecture == "Logulix" and cfg.vocab_size == 97
    assert cfg.embedding_scale == 0.7 and cfg.logit_scale == 1.3
    assert config_from_dict(cfg.to_dict()) == cfg
    assert [(i, n, f) for i, n, f in cfg.layer_runs()] == [
        (0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False),
        (1, 2, True), (2, 2, False), (3, None, False)]
    assert PL.layer_runs(L.L_MIXED) == [(i, f) for i, _, f in cfg.layer_runs()]
    plain = config_from_dict(L.L_PLAIN)
    assert plain.embedding_scale == 1.0 and plain.logit_scale == 1.0 and plain.loop is None


@pytest.mark.parametrize("change,word", [
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][0]["mixer"].update(vdim=8), "values are the keys"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda r: r["layers"][0]["mixer"].update(sink=4), "does not know"),
    (lambda r: r["layers"][2]["mixer"].update(decay=[0.5]), "one number a head"),
    (lambda r: r["layers"][1].update(type="mamba"), "not known"),
    (lambda r: r["layers"][0]["mlp"].update(kind="moe"), "not known"),
    (lambda r: r["loop"].update(stop=9), "not a run"),
    (lambda r: r.update(rope=1), "does not know"),
])
def test_config_refuses_what_it_does_not_know(change, word):
    raw = copy.deepcopy(L.L_MIXED)
    change(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_tensor_names_shapes_and_cache_specs():
    cfg = config_from_dict(L.L_MIXED)
    model = build_model(cfg)
    specs = model.tensor_specs()
    assert specs["embed"].shape == (97, 48) and specs["head"].shape == (97, 48)
    assert specs["loop.in"].shape == (48, 96) and specs["final.norm"].shape == (48,)
    assert specs["l0.mix.q"].shape == (64, 48) and specs["l0.mix.k"].shape == (32, 48)
    assert specs["l0.mix.q.conv"].shape == (64, 2) and specs["l0.mix.k.b"].shape == (32,)
    assert specs["l0.mix.o.b"].shape == (48,) and "l0.mix.v" not in specs
    assert specs["l1.mix.w1"].shape == (5, 48) and specs["l1.mix.w2"].shape == (48, 5)
    assert specs["l1.mix.u"].shape == (3, 16) and specs["l1.mix.mu.w"].shape == (48,)
    assert specs["l2.mix.v"].shape == (80, 48) and specs["l2.mix.o"].shape == (48, 80)
    assert "l1.norm2" not in specs and specs["l2.mlp.up"].shape == (40, 48)
    assert "l3.mix.q.norm" in specs and model.tied_names() == {}
    cache = model.cache_specs()
    assert len(cache) == 8                                   # 1 + 3 passes of 2 + 1
    assert cache[0] == PagedWithState(PagedKV(2, 16, 21), FixedState((96,), torch.float32))
    assert cache[1] == cache[3] == cache[5] == FixedState((3 * 16 * 16 + 48,), torch.float32)
    assert cache[2] == FixedState((2 * 24 * 40,), torch.float32)
    assert cache[7].paged == PagedKV(1, 32, 7) and cache[7].state.shape == (3 * 96,)
    # an attention without a convolution keeps pages only
    assert isinstance(build_model(config_from_dict(L.L_PLAIN)).cache_specs()[2], PagedKV)


def test_cache_manager_gives_a_paged_slot_its_state_too():
    model = build_model(config_from_dict(L.L_MIXED))
    cm = CacheManager(model.cache_specs(), num_blocks=6, block_size=4, max_requests=2,
                      max_seq_len=64, device="cpu")
    handles = cm.handles()
    assert handles[0].kind == "paged" and handles[0].state.shape == (2, 96)
    assert handles[0].k_pool.shape == (2, 6, 4, 16) and handles[0].window == 21
    assert handles[1].kind == "fixed" and handles[1].state.shape == (2, 3 * 16 * 16 + 48)
    assert handles[7].state.shape == (2, 288) and handles[7].k_pool.shape == (1, 6, 4, 32)
    assert cm.admit("a") and cm.reserve("a", 9)
    handles[0].state[cm.row("a")] = 1.0
    cm.commit("a", 9)
    cm.free("a")
    assert cm.admit("b") and cm.row("b") == 0
    assert handles[0].state[0].abs().max().item() == 0       # zeroed when claimed again
    cm.check()


def test_random_folder_and_shapes_give_the_decay_rank(tmp_path):
    raw = copy.deepcopy(L.L_PLAIN)
    cfg = config_from_dict(dict(raw, dtype="float32"))
    write_random_model(tmp_path / "m", cfg, 3)
    stored = json.loads((tmp_path / "m" / "config.json").read_text())
    stored["layers"][0]["mixer"].pop("rank")
    (tmp_path / "m" / "config.json").write_text(json.dumps(stored))
    bare = config_from_folder(tmp_path / "m")
    assert bare.layers[0]["mixer"].get("rank") is None
    with open_weights(tmp_path / "m") as f:
        full = bare.with_tensor_shapes({n: tuple(e.shape) for n, e in f.entries.items()})
    assert full.layers[0]["mixer"]["rank"] == 4 and full == cfg


def test_plain_mechanisms_on_hand_made_cases():
    """The oracle itself, on cases small enough to work out by hand."""
    u = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    y = PL.plain_causal_conv(u, torch.tensor([[10.0, 1.0]], dtype=torch.float64))
    assert y.flatten().tolist() == [1.0, 12.0, 24.0]
    x = torch.tensor([[[1.0, 0.0, 5.0, 0.0, 1.0, 7.0]]], dtype=torch.float64)
    pos = torch.tensor([1])
    # one pair a pairing, a quarter turn: base 1 makes every frequency 1
    import math
    q = PL.plain_rotate(x, 2, 1.0, 2.0 / math.pi, "interleaved", pos)
    assert torch.allclose(q[0, 0], torch.tensor([0.0, 1.0, 5.0, 0.0, 1.0, 7.0], dtype=torch.float64))
    q = PL.plain_rotate(x, 4, 1.0, 2.0 / math.pi, "half", pos)
    assert torch.allclose(q[0, 0], torch.tensor([-5.0, 0.0, 1.0, 0.0, 1.0, 7.0], dtype=torch.float64))
