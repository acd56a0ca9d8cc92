"""Host-side tests of the Zipedra design: its configuration, its description made of parts, the tensors it
expects, and properties of the plain implementation the GPU tests compare with."""
import copy

import pytest
import torch

import plain_zipedra
from zipedra_configs import CONFIGS, ZA, ZB, ZC


def test_the_registry_resolves_the_design_by_its_singular_key():
    from torchinferno_b200.config.registry import resolve_architecture, registered_architectures
    assert "Zipedra" in registered_architectures()
    assert resolve_architecture({"architecture": "Zipedra"}).name == "Zipedra"
    assert resolve_architecture({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    with pytest.raises(ValueError):
        resolve_architecture({"architecture": "Zipedra", "architectures": ["LlamaForCausalLM"]})


def test_config_errors_name_what_is_missing_or_wrong():
    from torchinferno_b200.config.model_config import ConfigError
    from torchinferno_b200.config.zipedra_config import ZipedraConfig
    ZipedraConfig.from_dict(ZA)
    for path, value in ((("width",), None), (("layers", 0, "mixer", "decay"), [0.5]), (("layers", 1, "mixer", "rot", "dims"), 3),
                        (("layers", 0, "type"), "conv"), (("loop", "stop"), 9), (("layers", 0, "mlp", "router", "top"), 6),
                        (("norm",), None), (("layers", 1, "mlp", "kind"), "glu")):
        bad = copy.deepcopy(ZA)
        node = bad
        for key in path[:-1]:
            node = node[key]
        if value is None:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        with pytest.raises(ConfigError):
            ZipedraConfig.from_dict(bad)


def test_the_schedule_gives_every_run_of_a_layer_its_own_cache_or_state():
    from torchinferno_b200.config.zipedra_config import ZipedraConfig
    from torchinferno_b200.models.spec import LayerCall, StageCall
    from torchinferno_b200.models.zipedra import build_zipedra
    spec = build_zipedra(ZipedraConfig.from_dict(ZA))
    calls = [(c.layer, c.cache) if isinstance(c, LayerCall) else ("stage", c.arg) for c in spec.schedule]
    assert calls == [("stage", 0), (0, None), (1, 0), ("stage", 1), (0, None), (1, 1), ("stage", 2), (0, None), (1, 2), (2, 3)]
    assert spec.cache_layers == 4 and spec.keeps_embedding_output and spec.logit_scale == 0.7
    spec = build_zipedra(ZipedraConfig.from_dict(ZB))
    assert [c.cache for c in spec.schedule] == [0, None, 1] and not spec.stages and not spec.keeps_embedding_output
    spec = build_zipedra(ZipedraConfig.from_dict(ZC))
    assert spec.cache_layers == 0 and [isinstance(c, StageCall) for c in spec.schedule] == [False, True, False, False]


def test_expected_tensors_and_requirements():
    from torchinferno_b200.weights.random_init import build_model
    model = build_model(ZA, dtype=torch.float32, device="cpu")
    names = model.expected_tensors()
    assert names["side.embed"].shape == (97, 30) and names["loop.in"].shape == (64, 128) and names["loop.step"].shape == (3, 64)
    assert names["l0.mlp.shared.sg"].shape == (1, 64) and names["l1.mix.dkv"].shape == (48, 64) and names["l1.mix.dkv.norm"].shape == (40,)
    assert names["l0.mix.norm"].shape == (72,) and names["l2.mix.uk"].shape == (24, 24) and "l2.mlp.up" not in names
    assert {"embed", "head", "final.norm", "l0.norm1", "l2.side.proj", "l0.mlp.e4.down", "l0.mlp.router"} <= set(names)
    caches, states = model.cache_requirements(), model.state_requirements()
    assert [(c.kv_heads, c.head_dim, c.value_width) for c in caches] == [(1, 48, 0)] * 3 + [(1, 28, 0)]
    assert [None if s is None else s.shape for s in states] == [None, (3, 16, 24), None, None, (3, 16, 24), None, None, (3, 16, 24), None, None]
    assert model.capturable()
    assert "l1.mlp.shared.up" not in build_model(ZB, dtype=torch.float32, device="cpu").expected_tensors() \
        and "side.embed" not in build_model(ZB, dtype=torch.float32, device="cpu").expected_tensors()


def test_a_random_model_folder_holds_exactly_the_expected_tensors(tmp_path):
    from torchinferno_b200.weights.random_init import build_model, write_random_model
    write_random_model(ZB, tmp_path, seed=3)
    config, weights = plain_zipedra.read_model_folder(tmp_path)
    assert set(weights) == set(build_model(ZB, dtype=torch.float32, device="cpu").expected_tensors())
    assert config["layers"] == ZB["layers"]


def test_state_slots_are_zeroed_for_a_new_request_and_keys_only_groups_take_pages():
    from torchinferno_b200.cache.manager import CacheManager
    from torchinferno_b200.parts.base import CacheSpec, StateSpec
    cache = CacheManager([CacheSpec(1, 12, None, value_dim=0)], [StateSpec((2, 3, 4)), None], page_size=4, num_pages=6,
                         max_requests=2, max_request_tokens=24, dtype=torch.float32, device="cpu")
    assert cache.groups[0].pool.shape == (1, 6, 4 * 12) and cache.kv_binding(0).keys.shape == (6, 1, 4, 12) and cache.kv_binding(0).values is None
    slot = cache.open("a")
    cache.extend("a", 9)
    cache.states[0][slot].fill_(7.0)
    cache.close("a")
    assert cache.open("b") == slot and float(cache.states[0][slot].abs().sum()) == 0.0
    cache.audit()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plain_implementation_is_causal_and_its_recurrence_matches_a_closed_form(name, tmp_path):
    from torchinferno_b200.weights.random_init import write_random_model
    config, seed = CONFIGS[name]
    write_random_model(config, tmp_path, seed=seed)
    cfg, w = plain_zipedra.read_model_folder(tmp_path)
    tokens = torch.randint(0, cfg["vocab"], (23,)).tolist()
    whole = plain_zipedra.forward(cfg, w, tokens)
    assert torch.isfinite(whole).all() and whole.abs().max() > 1e-3
    assert torch.allclose(plain_zipedra.forward(cfg, w, tokens[:9]), whole[:9], atol=1e-12, rtol=1e-10)
    # the linear attention recurrence against its sum form: o_t = sum_(s <= t) decay^(t - s) (q_t . k_s) v_s
    layer = next((i for i, l in enumerate(cfg["layers"]) if l["type"] == "lightning"), None)
    if layer is not None:
        m, p = cfg["layers"][layer]["mixer"], f"l{layer}.mix."
        h = torch.randn(13, cfg["width"], dtype=torch.float64)
        got = plain_zipedra.lightning_mixer(h, w, p, m, 1e-6)
        H, D, V = m["heads"], m["dim"], m["vdim"]
        q, k = (plain_zipedra.silu(h @ w[p + n].T).view(13, H, D) for n in ("q", "k"))
        v = plain_zipedra.silu(h @ w[p + "v"].T).view(13, H, V)
        t = torch.arange(13)
        power = (t[:, None] - t[None, :]).clamp(min=0).double()
        decay = torch.tensor(m["decay"], dtype=torch.float64)[:, None, None] ** power[None]
        decay = decay * (t[None, :, None] >= t[None, None, :])
        out = torch.einsum("hts,thd,shd,shv->thv", decay, q, k, v).reshape(13, H * V)
        want = (plain_zipedra.rms_norm(out, w[p + "norm"], 1e-6) * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T
        assert torch.allclose(got, want, atol=1e-10, rtol=1e-8)
