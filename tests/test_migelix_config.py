"""Reading, refusing and laying out Migelix configurations; runs without a GPU."""

import copy

import pytest
import torch

import migelix_cases as cases
from stride_b200.config import ConfigError, MigelixConfig, config_from_dict
from stride_b200.engine.loading import _declarations, footprint


def shapes_of(state):
    return {k: tuple(v.shape) for k, v in state.items()}


@pytest.mark.parametrize("case", sorted(cases.CASES))
def test_declarations_are_the_checkpoints_tensors(case):
    cfg = cases.CASES[case]
    state = cases.seeded_state(cfg, 1)
    config = config_from_dict(cfg, tensor_names=list(state), tensor_shapes=shapes_of(state))
    assert isinstance(config, MigelixConfig)
    declared = _declarations(config)
    assert set(declared) == set(state)
    for name, decl in declared.items():
        assert tuple(decl.shape) == tuple(state[name].shape), name
    again = config_from_dict(config.to_dict())           # the ranks now stand in the dictionary
    assert again == config and _declarations(again).keys() == declared.keys()


def test_layers_that_share_weights_run_on_caches_of_their_own():
    spec = config_from_dict(cases.CASE_A, ["x"], shapes_of(cases.seeded_state(cases.CASE_A, 1))).to_model_spec()
    assert len(spec.layers) == 3 and [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (0, 3), (2, 4)]
    assert spec.num_cache_slots == 5 and all(e.writes_cache for e in spec.schedule)
    left = dict(spec.layers[0].mixer.params)["branches"][0][0]
    assert left.kind == "attention" and left.window == 21 and left.bias and dict(left.params)["values"] == "keys"
    assert dict(left.position.params)["rotated"] == 16 and left.position.scaling.rope_type == "yarn"
    assert dict(spec.head_spec().params)["softcap"] == 6.0 and spec.head_spec().name is None


def test_low_ranks_come_from_the_checkpoint_or_the_dictionary():
    cfg = cases.CASE_A
    state = cases.seeded_state(cfg, 1, decay_rank=3, gate_rank=9, shift_rank=4)
    config = config_from_dict(cfg, list(state), shapes_of(state))
    assert config.layers[0]["mixer"]["right"]["decay_rank"] == 3 and config.layers[0]["mixer"]["right"]["gate_rank"] == 9
    assert config.layers[1]["mixer"]["decay_rank"] == 4 and config.layers[3]["mixer"]["right"]["decay_rank"] == 3
    with pytest.raises(ValueError, match="decay_rank"):      # neither a checkpoint nor a key: the parts cannot be sized
        _declarations(config_from_dict(cfg))
    given = config_from_dict(cases.CASE_D)                   # case D names its ranks
    assert _declarations(given)["l1.mix.right.a1"].shape == (4, 100)


def test_footprint_counts_pages_and_state():
    cfg = cases.CASE_B
    state = cases.seeded_state(cfg, 1)
    f = footprint(config_from_dict(cfg, list(state), shapes_of(state)), "bfloat16")
    # pages: layer 0 keeps keys and values of 1 x 48, layer 2 of 2 x 16; state: wkv 64 x 64 + width (twice), delta 2 x 8 x 16 and no tail
    assert f["kv_bytes_per_token"] == 2 * (2 * 48 + 2 * 2 * 16)
    assert f["state_bytes_per_request"] == 4 * (2 * (64 * 64 + 80) + 2 * 8 * 16)


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(vdim=8), "vdim"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=2), "group"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=15), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=34), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(kv_heads=3), "group"),
    (lambda d: d["layers"][3].update(weights_of=4), "tensors of its own"),
    (lambda d: d["layers"][3].update(weights_of=3), "another layer"),
    (lambda d: d["layers"][3]["mixer"].update(left_scale=0.1), "must equal"),
    (lambda d: d["layers"][2]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda d: d["layers"][0].update(mlp={"kind": "moe"}), "dense"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.update(vocab=0), "vocab"),
])
def test_what_is_refused(change, message):
    d = copy.deepcopy(cases.CASE_A)
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_head_order_for_neighbour_pairs():
    """Turned pairs go to (i, i + half); entries that pass unchanged fill both halves behind them."""
    from stride_b200.config import PositionSpec
    from stride_b200.parts import Runtime, build_part
    rt = Runtime("meta", torch.float32, 1, 1)
    part = build_part("position", PositionSpec("rope", head_dim=8, theta=100.0, max_positions=4, params=(("pairing", "neighbours"), ("rotated", 4))), rt)
    assert part.head_permutation() == [0, 2, 4, 5, 1, 3, 6, 7]
    whole = build_part("position", PositionSpec("rope", head_dim=6, theta=100.0, max_positions=4, params=(("pairing", "neighbours"),)), rt)
    assert whole.head_permutation() == [0, 2, 4, 1, 3, 5]
    plain_halves = build_part("position", PositionSpec("rope", head_dim=6, theta=100.0, max_positions=4), rt)
    assert plain_halves.head_permutation() is None
