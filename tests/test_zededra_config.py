"""Zededra without a GPU: configuration, registry, tensor names, cache slots, the
state's layout, and the plain implementation against itself (token by token with the
state carried against whole sequences)."""

import copy

import pytest
import torch

import plain_zededra as PZ
import tiny_zededra as Z
from mini_llm_stack_b200.cache.manager import CacheManager
from mini_llm_stack_b200.config import (ConfigError, ZededraConfig, build_model, config_from_dict,
                                        config_from_folder)
from mini_llm_stack_b200.parts import FixedState, PagedKV
from mini_llm_stack_b200.parts.mlstm import state_columns


def test_config_round_trip_and_registry(tmp_path):
    cfg = config_from_dict(Z.Z_MIXED)
    assert isinstance(cfg, ZededraConfig) and cfg.vocab_size == 97 and cfg.norm_eps == 1e-5
    assert cfg.to_dict() == Z.Z_MIXED
    assert config_from_dict(cfg.to_dict()) == cfg
    Z.make_zededra(tmp_path / "m", Z.Z_PLAIN, 1, "float32")
    assert config_from_folder(tmp_path / "m").to_dict() == dict(Z.Z_PLAIN, dtype="float32")


def test_layer_runs_follow_the_loop():
    cfg = config_from_dict(Z.Z_MIXED)
    runs = cfg.layer_runs()
    assert [r[0] for r in runs] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    assert [(r[1], r[2]) for r in runs if r[2]] == [(0, True), (1, True), (2, True)]
    assert runs == PZ.layer_runs(Z.Z_MIXED)
    assert [r[0] for r in config_from_dict(Z.Z_PLAIN).layer_runs()] == [0, 1]


@pytest.mark.parametrize("change, word", [
    (lambda c: c.update(rope=1), "does not know"),
    (lambda c: c["layers"][0].update(type="conv"), "not known"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "lacks"),
    (lambda c: c["layers"][1]["mixer"].update(window=4), "does not know"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "not known"),
    (lambda c: c["loop"].update(stop=9), "not a run"),
    (lambda c: c.pop("norm"), "lacks"),
])
def test_config_errors_name_the_key(change, word):
    raw = copy.deepcopy(Z.Z_MIXED)
    change(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_tensor_names_and_cache_slots():
    model = build_model(config_from_dict(Z.Z_MIXED))
    names = set(model.tensor_specs())
    assert {"embed", "loop.step", "final.norm", "l0.norm1", "l0.mix.dq.norm", "l0.mlp.gate",
            "l1.mix.i.b", "l1.mlp.router", "l1.mlp.e4.down", "l1.mlp.shared.up", "l2.norm1",
            "l3.mlp.e2.gate"} <= names
    assert "l2.norm2" not in names and "l3.mlp.shared.up" not in names   # no feed-forward; no shared expert
    assert model.tensor_specs()["loop.step"].shape == (3, 48)
    specs = model.cache_specs()
    assert len(specs) == 11                                  # one slot a layer run
    assert specs[0] == PagedKV(1, 48, None, shared_kv=True)  # a latent of 40 in rows of 48
    assert specs[1] == FixedState((2, 24 * 40 + 24 + 3), torch.float32)  # 40 columns: three groups
    assert specs[3] == FixedState((4, 8 * 80 + 8 + 5), torch.float32)    # 80 columns: five groups
    assert specs[1] == specs[4] == specs[7]                  # every pass its own slot, same shape
    # the cache manager groups them: latents of equal width share pages, every pass has its own pool
    cache = CacheManager(specs, num_blocks=4, block_size=8, max_requests=2, max_seq_len=32,
                         allocate=True)
    assert sorted(len(g.members) for g in cache.paged) == [1, 1, 3]
    assert all(g.kv.shape[1] == 1 for g in cache.paged)      # one pool is keys and values
    assert sorted(len(g.members) for g in cache.fixed) == [3, 3]


def test_state_columns_leave_a_thread_at_most_64_rows():
    for e, f in [(8, 80), (32, 48), (256, 512), (1024, 64), (40, 150), (4096, 16)]:
        fc = state_columns(e, f)
        assert 1 <= fc <= min(f, 16) and -(-e // (256 // fc)) <= 64


def test_plain_mlstm_carries_its_state():
    raw = Z.one_layer({"type": "mlstm", "mixer": Z.mlstm(2, 6, 10, 5.0), "mlp": None})
    m = raw["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(2)
    w = {f"p.{n}": torch.randn(s, generator=g, dtype=torch.float64) * 0.3 for n, s in
         [("q", (12, 16)), ("k", (12, 16)), ("v", (20, 16)), ("g", (20, 16)), ("o", (16, 20)),
          ("norm", (20,)), ("i", (2, 16)), ("i.b", (2,)), ("f", (2, 16)), ("f.b", (2,))]}
    h = torch.randn(9, 16, generator=g, dtype=torch.float64)
    whole, _ = PZ.plain_mlstm(h, w, "p", m, 1e-5)
    state, rows = None, []
    for cut in ((0, 4), (4, 5), (5, 9)):
        y, state = PZ.plain_mlstm(h[cut[0]:cut[1]], w, "p", m, 1e-5, state)
        rows.append(y)
    assert torch.allclose(torch.cat(rows), whole, atol=1e-12)


def test_plain_router_weighs_inputs_not_outputs():
    g = torch.Generator().manual_seed(4)
    w = {"p.router": torch.randn(3, 8, generator=g, dtype=torch.float64)}
    for i in range(3):
        w[f"p.e{i}.gate"] = torch.randn(5, 8, generator=g, dtype=torch.float64)
        w[f"p.e{i}.up"] = torch.randn(5, 8, generator=g, dtype=torch.float64)
        w[f"p.e{i}.down"] = torch.randn(8, 5, generator=g, dtype=torch.float64)
    h = torch.randn(4, 8, generator=g, dtype=torch.float64)
    out = PZ.plain_routed_experts(h, w, "p", Z.moe(3, 2, 5))
    idx, val = PZ.plain_route(h, w["p.router"], 2)
    t = 1
    want = sum(PZ.plain_silu_glu((val[t, j].double() * h[t])[None], w, f"p.e{int(idx[t, j])}")[0]
               for j in range(2))
    assert torch.allclose(out[t], want, atol=1e-12)
    scaled_after = sum(val[t, j].double() * PZ.plain_silu_glu(h[t][None], w, f"p.e{int(idx[t, j])}")[0]
                       for j in range(2))
    assert not torch.allclose(out[t], scaled_after, atol=1e-3)
