"""Configuration of the Nidilix decoder: what config.json gives is read, checked and laid out as parts; no GPU."""

import copy

import pytest

import nidilix_cases as cases


def test_the_registry_places_the_architecture_by_its_singular_key():
    from stride_b200.config import NidilixConfig, config_from_dict, registered_architectures
    assert "Nidilix" in registered_architectures()
    cfg = config_from_dict(cases.CASE_A)
    assert isinstance(cfg, NidilixConfig) and cfg.width == 96 and cfg.vocab == 211 and cfg.side_dim == 12
    assert config_from_dict(cfg.to_dict()) == cfg
    assert config_from_dict(dict(cases.CASE_A, architectures=["Nidilix"])) == cfg


def test_layers_become_parts_and_a_borrowed_cache_becomes_a_shared_slot():
    from stride_b200.config import config_from_dict
    spec = config_from_dict(cases.CASE_B).to_model_spec()
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["latent_attention", "latent_attention", "rglru", "latent_attention", "rglru"]
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False), (4, 4, True)]
    assert spec.layers[1].feed_forward is None and spec.layers[1].ffn_norm is None and spec.layers[1].after == ()
    assert spec.layers[0].mixer_norm.kind == "dyt" and spec.final_norm.prefix == "final.norm"
    assert dict(spec.layers[3].mixer.params)["own_latent"] is False
    assert spec.layers[0].mixer.position.head_dim == 6 and dict(spec.layers[0].mixer.params)["rot_dim"] == 12
    assert dict(spec.layers[2].feed_forward.params) == {"experts": 7, "top": 1, "shared": 48, "router_bias": True}
    side = config_from_dict(cases.CASE_A).to_model_spec().layers[2].after[0]
    assert (side.kind, side.dim, side.offset, side.table_width, side.table_name) == ("token_side", 12, 24, 48, "side.embed")


def test_declared_tensors_are_the_checkpoint_names():
    from stride_b200.config import config_from_dict
    from stride_b200.engine.loading import _declarations, footprint
    for cfg in cases.CASES.values():
        declared = _declarations(config_from_dict(cfg))
        state = cases.seeded_state(cfg, 1)
        assert set(declared) == set(state)
        for name, decl in declared.items():
            assert tuple(decl.shape) == tuple(state[name].shape), name
    f = footprint(config_from_dict(cases.CASE_B), "bfloat16")
    assert f["kv_bytes_per_token"] == 2 * ((24 + 12) + (56 + 4))          # two caches; the borrowing layer adds nothing
    assert f["state_bytes_per_request"] == 4 * (1 * 80 + 7 * 64)           # taps rows of width each


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][3]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=0), "latent_attention layer"),
    (lambda d: d["layers"][3]["mixer"].update(kv_rank=48), "must equal"),
    (lambda d: d["layers"][0]["mixer"].update(blocks=7), "equal blocks"),
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=6), "exceeds"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "routed mixture"),
    (lambda d: d.pop("residual_mult"), "residual_mult"),
    (lambda d: d["norm"].pop("eps"), "eps"),
])
def test_what_does_not_fit_is_refused(change, message):
    from stride_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(cases.CASE_A)
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_a_model_folder_is_written_and_read_back(tmp_path):
    from stride_b200.config import config_from_dict, load_config
    from stride_b200.engine.loading import write_random_model
    from stride_b200.weights import SafetensorsSource, check_source
    from stride_b200.engine.loading import _declarations
    cfg = config_from_dict(cases.CASE_C)
    folder = write_random_model(cfg, 5, str(tmp_path / "m"))
    source = SafetensorsSource(folder)
    again = load_config(folder, tensor_names=source.names())
    assert again == cfg
    check_source(source, _declarations(again), ())
    assert source.describe("l0.norm1.alpha")[0] == ()


def test_presets_of_the_design_parse_and_plan():
    from stride_b200.config import config_from_dict, plan_memory, preset
    tiny = config_from_dict(preset("nidilix-tiny"))
    assert [l["type"] for l in tiny.layers] == ["rglru", "latent_attention", "rglru", "latent_attention"] and tiny.layers[3]["mixer"]["kv_from"] == 1
    big = config_from_dict(preset("nidilix-2048"))
    plan = plan_memory(big, "bfloat16", 180 * (1 << 30), 16, 0.15, name="nidilix-2048")
    assert plan.concurrent_sequences(8192) > 0
