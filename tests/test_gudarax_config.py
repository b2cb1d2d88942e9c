"""Gudarax on the host: the configuration's checks, the plan, the cache groups and state that follow from it, and the plain
statement's own pieces."""
import copy

import pytest
import torch

import plain_gudarax as plain
from gudarax_configs import CONFIGS


def typed(raw):
    from wllm_b200.config import GudaraxConfig
    return GudaraxConfig.from_dict(raw, where="test")


def model_of(raw, dtype=torch.bfloat16):
    from wllm_b200.config import resolve_architecture
    from wllm_b200.engine.model import ComposedModel
    arch = resolve_architecture("Gudarax")
    return ComposedModel(arch.make_plan(typed(raw)), dtype)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_round_trip_and_defaults(name):
    cfg = typed(CONFIGS[name])
    again = typed(cfg.to_dict())
    assert again == cfg
    for layer, raw in zip(cfg.layers, CONFIGS[name]["layers"]):
        m = layer["mixer"]
        if layer["type"] == "attention":
            assert m["kv_heads"] == raw["mixer"].get("kv_heads", m["heads"]) and m["vdim"] == raw["mixer"].get("vdim", m["dim"])
            assert m["scale"] == raw["mixer"].get("scale", m["dim"] ** -0.5) and m["v_mix"] == raw["mixer"].get("v_mix", False)
    assert cfg.side_dim == (CONFIGS[name].get("token_side") or {}).get("dim")
    assert cfg.embedding_scale == (CONFIGS[name].get("embedding") or {}).get("scale", 1.0)


def test_every_problem_is_named_at_once():
    from wllm_b200.config import ConfigError
    raw = copy.deepcopy(CONFIGS["mixed"])
    del raw["vocab"]
    raw["layers"][0]["type"] = "conv"
    raw["layers"][1]["mixer"]["kv_heads"] = 3
    raw["layers"][2]["mlp"]["router"]["top"] = 9
    raw["layers"][3]["mixer"]["vdim"] = 8           # its values cannot be blended with the first such layer's
    del raw["layers"][5]["mixer"]["conv"]
    with pytest.raises(ConfigError) as e:
        typed(raw)
    text = str(e.value)
    for piece in ("vocab", "layers[0].type", "4 heads are no multiple of 3", "top 9 of 6", "cannot be mixed", "conv"):
        assert piece in text, (piece, text)


def test_the_plan_names_every_tensor_and_no_other():
    model = model_of(CONFIGS["mixed"])
    names = {ps.name: ps for ps in model.param_specs()}
    assert {"embed", "pos", "side.embed", "final.norm", "head"} <= set(names)
    assert names["side.embed"].shape == (200, 6 * 8) and names["pos"].shape == (400, 64)
    assert names["l1.mix.vmix"].shape == () and names["l3.mix.vmix"].shape == () and "l4.mix.vmix" not in names
    assert names["l1.mix.q.b"].shape == (64,) and names["l1.mix.v.b"].shape == (48,) and names["l1.mix.q.norm"].shape == (64,)
    assert names["l2.mix.dq"].shape == (24, 64) and names["l2.mix.uq"].shape == (64, 24) and names["l2.mix.g"].shape == (48, 64)
    assert names["l0.mix.q.conv"].shape == (32, 4) and names["l0.mix.v.conv"].shape == (96, 4) and names["l0.mix.A_log"].shape == (4,)
    assert names["l0.mlp.e5.up"].shape == (40, 64) and "l0.mlp.e0.gate" not in names and names["l0.mlp.router"].shape == (6, 64)
    assert "l3.norm2" not in names and "l3.side.norm" in names
    bare = {ps.name for ps in model_of(CONFIGS["bare"]).param_specs()}
    assert not any("side" in n for n in bare) and not any(n.endswith("vmix") for n in bare)


def test_cache_groups_and_state_follow_from_the_mixers():
    model = model_of(CONFIGS["mixed"])
    groups = {g.name: g for g in model.group_specs}
    assert set(groups) == {"window21-2x16v24", "all-1x32-in-keys", "window40-2x32v24", "all-2x16"}
    states = {s.name: tuple(s.shape) for s in model.state_specs}
    assert states == {"run0.state": (4, 16, 24), "run0.conv": (3, 2 * 32 + 96), "run5.state": (2, 24, 16), "run5.conv": (2, 2 * 48 + 32)}
    assert {s.name for s in model_of(CONFIGS["bare"]).state_specs} == {"run1.state"}          # one tap: no inputs are kept
    roles = [b.mixer.value_mix["role"] for b in model.blocks if getattr(b.mixer, "value_mix", None)]
    assert roles == ["first", "later"]
    assert model.graph_safe


def test_slopes_masks_and_the_short_convolution_of_the_plain_statement():
    from wllm_b200.models.gudarax import distance_slopes
    assert distance_slopes(8) == [2.0 ** -(h + 1) for h in range(8)]
    assert torch.allclose(plain.slopes(4, torch.float64), torch.tensor([0.25, 0.0625, 2.0 ** -6, 2.0 ** -8], dtype=torch.float64))
    seen = plain.window_visible(6, 3)
    assert seen[5].tolist() == [False, False, False, True, True, True] and seen[1].tolist() == [True, True, False, False, False, False]
    assert plain.window_visible(4, None)[3].all()
    x = torch.arange(1.0, 6.0)[:, None]
    taps = torch.tensor([[100.0, 10.0, 1.0]])
    assert plain.short_conv(x, taps)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]       # the last tap is the token's own
    # the delta rule with beta = 1 and no decay stores v along k and reads it back along q = k
    w = {"q": torch.eye(2), "k": torch.eye(2), "v": torch.eye(2), "q.conv": torch.ones(2, 1), "k.conv": torch.ones(2, 1), "v.conv": torch.ones(2, 1),
         "b": torch.zeros(1, 2), "a": torch.zeros(1, 2), "A_log": torch.tensor([-30.0]), "dt_bias": torch.zeros(1), "norm": torch.ones(2),
         "g": torch.eye(2), "o": torch.eye(2)}
    out = plain.delta({"heads": 1, "dim": 2, "vdim": 2, "conv": 1}, w, "", torch.tensor([[3.0, 0.0], [3.0, 0.0]]), 1e-6)
    assert out.shape == (2, 2) and out[1, 0] > out[0, 0] > 0
