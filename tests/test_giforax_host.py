"""Host-side tests of the Giforax design: its configuration, its description made of parts, the tensors it expects,
and properties of the plain implementation the GPU tests compare with."""
import copy

import pytest
import torch

import plain_giforax
from giforax_configs import CONFIGS, GA, GB, GC, GD, GE


def test_the_registry_resolves_the_design():
    from torchinferno_b200.config.registry import registered_architectures, resolve_architecture
    assert "Giforax" in registered_architectures()
    assert resolve_architecture({"architecture": "Giforax"}).name == "Giforax"
    with pytest.raises(ValueError):
        resolve_architecture({"architecture": "Giforax", "architectures": ["LlamaForCausalLM"]})


def test_config_errors_name_what_is_missing_or_wrong():
    from torchinferno_b200.config.giforax_config import GiforaxConfig
    from torchinferno_b200.config.model_config import ConfigError
    for config in (GA, GB, GC, GD, GE):
        GiforaxConfig.from_dict(config)
    for path, value in ((("width",), None), (("embedding",), None), (("norm", "eps"), 0.0), (("layers", 0, "type"), "conv"),
                        (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 18),
                        (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "mask"), None),
                        (("layers", 2, "mixer", "kv_from"), 2), (("layers", 2, "mixer", "kv_from"), 1),
                        (("layers", 2, "mixer", "vdim"), 16), (("layers", 0, "mlp", "router", "top"), 4),
                        (("layers", 0, "mlp", "expert", "limit"), None), (("layers", 1, "mlp", "kind"), "dense"),
                        (("layers", 1, "mixer", "width"), 0)):
        bad = copy.deepcopy(GA)
        node = bad
        for key in path[:-1]:
            node = node[key]
        if value is None:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        with pytest.raises(ConfigError):
            GiforaxConfig.from_dict(bad)
    chained = copy.deepcopy(GB)         # a layer may not read the keys of a layer that has none of its own
    chained["layers"][3]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError):
        GiforaxConfig.from_dict(chained)


def test_the_schedule_shares_cache_layers_and_gives_recurrences_state():
    from torchinferno_b200.config.giforax_config import GiforaxConfig
    from torchinferno_b200.models.giforax import build_giforax
    spec = build_giforax(GiforaxConfig.from_dict(GA))
    assert [(c.layer, c.cache, c.writes_cache) for c in spec.schedule] == [(0, 0, True), (1, None, True), (2, 0, False), (3, 1, True)]
    assert spec.cache_layers == 2 and spec.history_depth == 6 and spec.embedding_scale == 3.0
    spec = build_giforax(GiforaxConfig.from_dict(GB))
    assert [(c.cache, c.writes_cache) for c in spec.schedule] == [(None, True), (0, True), (0, False), (0, False)]
    assert build_giforax(GiforaxConfig.from_dict(GC)).cache_layers == 0


def test_expected_tensors_and_requirements():
    from torchinferno_b200.weights.random_init import build_model
    model = build_model(GA, dtype=torch.float32, device="cpu")
    names = model.expected_tensors()
    assert names["l0.mix.q"].shape == (64, 64) and names["l0.mix.k"].shape == (32, 64) and names["l0.mix.v"].shape == (48, 64)
    assert names["l0.mix.g"].shape == (4, 64) and names["l0.mix.pb"].shape == (4,) and names["l0.mix.o"].shape == (64, 96)
    assert "l2.mix.k" not in names and "l2.mix.v" not in names and "l2.norm2" not in names and "l2.mlp.router" not in names
    assert names["l1.mix.z.b"].shape == (72,) and names["l1.mix.x"].shape == (72, 64) and names["l1.mix.o"].shape == (64, 72)
    assert names["l0.mlp.e2.gate"].shape == (24, 64) and names["l0.mlp.shared.down"].shape == (64, 40) and "l1.mlp.shared.up" not in names
    assert [names[f"l{i}.dwa"].shape for i in range(4)] == [(2,), (3,), (4,), (5,)]
    assert {"embed", "head", "final.norm", "final.norm.b", "l3.norm2b.b", "l0.norm1b"} <= set(names)
    caches, states = model.cache_requirements(), model.state_requirements()
    assert [(c.kv_heads, c.head_dim, c.value_width) for c in caches] == [(2, 16, 24), (2, 8, 8)]
    assert [None if s is None else s.shape for s in states] == [None, (72,), None, None]
    assert model.capturable()


def test_a_random_model_folder_holds_exactly_the_expected_tensors(tmp_path):
    from torchinferno_b200.weights.random_init import build_model, write_random_model
    write_random_model(GB, tmp_path, seed=3)
    config, weights = plain_giforax.read_model_folder(tmp_path)
    assert set(weights) == set(build_model(GB, dtype=torch.float32, device="cpu").expected_tensors())
    assert config["layers"] == GB["layers"]
    assert float((weights["l1.norm1"] - 1).abs().max()) > 0.01 and float(weights["l1.norm1.b"].abs().max()) > 0.01


def test_keys_and_values_of_different_widths_share_a_page_and_groups_follow_shapes():
    from torchinferno_b200.cache.manager import CacheManager
    from torchinferno_b200.weights.random_init import build_model
    model = build_model(GA, dtype=torch.float32, device="cpu")
    cache = CacheManager(model.cache_requirements(), model.state_requirements(), page_size=4, num_pages=6, max_requests=2,
                         max_request_tokens=24, dtype=torch.float32, device="cpu")
    assert len(cache.groups) == 2
    b = cache.kv_binding(0)
    assert b.keys.shape == (6, 2, 4, 16) and b.values.shape == (6, 2, 4, 24) and b.keys.stride(0) == b.values.stride(0) == 4 * 2 * 40
    slot = cache.open("a")
    cache.states[1][slot].fill_(3.0)
    cache.close("a")
    assert cache.open("b") == slot and float(cache.states[1][slot].abs().sum()) == 0.0
    cache.audit()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plain_implementation_is_causal_and_respects_chunks(name, tmp_path):
    from torchinferno_b200.weights.random_init import write_random_model
    config, seed = CONFIGS[name]
    write_random_model(config, tmp_path, seed=seed)
    cfg, w = plain_giforax.read_model_folder(tmp_path)
    tokens = torch.randint(0, cfg["vocab"], (53,)).tolist()
    whole = plain_giforax.forward(cfg, w, tokens)
    assert torch.isfinite(whole).all() and whole.abs().max() > 1e-3
    assert torch.allclose(plain_giforax.forward(cfg, w, tokens[:19]), whole[:19], atol=1e-12, rtol=1e-10)


def test_plain_mechanisms_against_closed_forms():
    g = torch.Generator().manual_seed(5)
    # chunks: a query sees back to the start of its own run of positions and no further
    seen = plain_giforax.visible(torch.arange(10), 4)
    assert seen[5].tolist() == [False] * 4 + [True, True] + [False] * 4 and seen[4].tolist() == [False] * 4 + [True] + [False] * 5
    assert seen[3].tolist() == [True] * 4 + [False] * 6 and seen[8].tolist() == [False] * 8 + [True, False]
    # the recurrence against its closed sum: S_t = sum_s z_s c_s prod_(s < r <= t) (1 - z_r)
    m, W = {"width": 6}, 5
    w = {"p.z": torch.randn(6, W, generator=g).double(), "p.z.b": torch.randn(6, generator=g).double(),
         "p.x": torch.randn(6, W, generator=g).double(), "p.x.b": torch.randn(6, generator=g).double(),
         "p.g": torch.randn(6, W, generator=g).double(), "p.o": torch.eye(6, dtype=torch.float64)}
    h = torch.randn(9, W, generator=g).double()
    got, last = plain_giforax.min_gru_mixer(h, w, "p.", m)
    z = torch.sigmoid(h @ w["p.z"].T + w["p.z.b"])
    u = h @ w["p.x"].T + w["p.x.b"]
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.stack([sum(z[s] * c[s] * torch.prod(1 - z[s + 1:t + 1], dim=0) for s in range(t + 1)) for t in range(9)])
    gate = h @ w["p.g"].T
    assert torch.allclose(got, S * gate * torch.sigmoid(gate), atol=1e-12) and torch.allclose(last, S[-1], atol=1e-12)
    # carried state: two halves give what the whole gives
    first, state = plain_giforax.min_gru_mixer(h[:4], w, "p.", m)
    second, _ = plain_giforax.min_gru_mixer(h[4:], w, "p.", m, state)
    assert torch.allclose(torch.cat([first, second]), got, atol=1e-12)
    # the candidate is continuous at 0 and the gated unit respects its limit
    assert abs(float(torch.sigmoid(torch.tensor(0.0, dtype=torch.float64))) - 0.5) < 1e-12
    w2 = {"e.gate": torch.full((1, 1), 10.0).double(), "e.up": torch.full((1, 1), -10.0).double(), "e.down": torch.ones(1, 1).double()}
    y = plain_giforax.gated_unit(torch.ones(1, 1).double(), w2, "e.", 2.0)
    assert abs(float(y) - 2.0 * float(torch.sigmoid(torch.tensor(2.0 * 1.702, dtype=torch.float64))) * (-2.0 + 1)) < 1e-12
