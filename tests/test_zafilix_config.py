"""Zafilix on the host: reading config.json, the plan's tensors and runs, cache groups (blocks, windows, rows that hold keys
and values at once), the pages that a mask of blocks gives back, and the plain statement's own masks and turns."""
import copy
import json

import pytest
import torch

import plain_zafilix as plain
from zafilix_configs import CONFIGS, HEADS64, MIXED, ODD, WHOLE
from wllm_b200.cache import CacheGroupSpec, CacheManager
from wllm_b200.config import ConfigError, ZafilixConfig, resolve_architecture
from wllm_b200.engine import ComposedModel


def model_of(raw):
    cfg = ZafilixConfig.from_dict(raw)
    return cfg, ComposedModel(resolve_architecture("Zafilix").make_plan(cfg), torch.float32)


def test_a_round_trip_through_a_dictionary_keeps_everything():
    for raw in CONFIGS.values():
        cfg = ZafilixConfig.from_dict(raw)
        assert ZafilixConfig.from_dict(cfg.to_dict()) == cfg
        assert json.loads(json.dumps(cfg.to_dict()))["architecture"] == "Zafilix"


@pytest.mark.parametrize("damage,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].__setitem__("type", "retention"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("factor"), "factor"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 10), "rot"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "experts"), "kind"),
    (lambda c: c["layers"][4].__setitem__("weights_of", 4), "weights_of"),
    (lambda c: c["layers"][5].__setitem__("weights_of", 4), "tensors of its own"),
    (lambda c: c["layers"][4]["mixer"]["mask"].__setitem__("size", 22), "equal"),
])
def test_a_bad_config_is_refused_with_the_key_named(damage, word):
    raw = copy.deepcopy(MIXED)
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        ZafilixConfig.from_dict(raw)


def test_what_a_file_leaves_out_does_not_exist():
    cfg = ZafilixConfig.from_dict(WHOLE)
    assert cfg.embedding_scale == 1.0 and cfg.logit_scale == 1.0
    assert ZafilixConfig.from_dict(ODD).logit_softcap is None
    assert "mask" not in cfg.layers[0]["mixer"] and "rot" not in cfg.layers[2]["mixer"]
    assert cfg.layers[1]["mixer"]["kv_heads"] == 3 and cfg.layers[1]["mixer"]["vdim"] == 16
    assert cfg.layers[1]["mixer"]["scale"] == 16 ** -0.5 and cfg.layers[0]["mixer"]["scale"] == 16 ** -0.5
    _, model = model_of(WHOLE)
    assert [g.window for g in model.group_specs] == [None] * len(model.group_specs)


def test_the_plan_names_every_tensor_once_and_a_layer_on_anothers_tensors_names_none():
    cfg, model = model_of(MIXED)
    names = [p.name for p in model.param_specs()]
    assert len(names) == len(set(names))
    assert not [n for n in names if n.startswith(("l4.", "l5.", "l6."))]
    assert {"l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.g", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv", "l2.norm1",
            "l0.mlp.up", "l0.mlp.down", "final.norm", "head", "embed"} <= set(names)
    assert "l2.norm2" not in names and "l2.mlp.up" not in names          # layer 2 has no feed-forward
    shapes = {p.name: tuple(p.shape) for p in model.param_specs()}
    assert shapes["l0.mix.q.norm"] == (64,) and shapes["l0.mix.k.norm"] == (32,) and shapes["l0.mix.g"] == (96, 64)
    assert shapes["l1.mix.q"] == (4 * 24, 64) and shapes["l1.mix.dkv"] == (40, 64) and shapes["l1.mix.uk"] == (64, 32)
    assert shapes["l1.mix.uv"] == (48, 32) and shapes["l1.mix.o"] == (64, 48)
    assert [r.block for r in model.plan.runs] == [0, 1, 2, 3, 1, 0, 2] and len(model.blocks) == 4
    assert [cfg.owner(i) for i in range(7)] == [0, 1, 2, 3, 1, 0, 2]


def test_every_run_has_a_cache_of_its_own_in_the_group_of_its_mask():
    _, model = model_of(MIXED)
    by_name = {g.name: g for g in model.group_specs}
    assert set(by_name) == {"blocks24-2x16v24", "window21-1x40v32-in-keys", "window40-1x56v40-in-keys", "blocks70-1x32"}
    assert by_name["blocks24-2x16v24"].layers == 2 and by_name["window21-1x40v32-in-keys"].layers == 2
    assert by_name["window40-1x56v40-in-keys"].layers == 2 and by_name["blocks70-1x32"].layers == 1
    assert by_name["blocks24-2x16v24"].blocks and not by_name["window21-1x40v32-in-keys"].blocks
    assert by_name["window21-1x40v32-in-keys"].values_in_keys and by_name["window21-1x40v32-in-keys"].kv_heads == 1
    refs = [(r.group, r.layer) for r in model.cache_refs]
    assert len(set(refs)) == 7 and all(r.writes for r in model.cache_refs)
    # a latent row is held in steps of 8 elements: 20 + 6 -> 32
    _, odd = model_of(ODD)
    assert {g.name for g in odd.group_specs} == {"window17-1x32v20-in-keys", "blocks16-1x16v8"}


def test_a_group_of_rows_that_hold_keys_and_values_has_one_pool():
    spec = CacheGroupSpec("w", 2, 1, 40, 21, 32, 0, False, True)
    cm = CacheManager([spec], page_size=8, num_pages=4, max_requests=2, dtype=torch.float32, device="cpu")
    g = cm.groups[0]
    assert g.keys(1).data_ptr() == g.values(1).data_ptr() and g.keys(1).shape == (4, 1, 8, 40)
    assert g.bytes_per_token() == 2 * 40 * 4


@pytest.mark.parametrize("size,page", [(24, 8), (16, 16), (10, 4), (70, 16), (5, 8)])
def test_blocks_give_back_the_pages_in_front_of_the_block_the_next_token_lies_in(size, page):
    spec = CacheGroupSpec("b", 1, 1, 8, size, None, 0, True, False)
    assert [spec.first_needed(n) for n in (0, size - 1, size, size + 1, 3 * size - 1, 3 * size)] == [0, 0, size, size, 2 * size, 3 * size]
    cm = CacheManager([spec], page_size=page, num_pages=64, max_requests=2, dtype=torch.float32, device=None)
    rc = cm.open("a")
    held = []
    for n in (3, size, 1, 2 * size + 1, 1, 1, size):
        cm.reserve([(rc, n)])
        cm.commit(rc, n)
        first = rc.num_tokens - rc.num_tokens % size
        table = rc.tables[0]
        assert all((p < 0) == ((i + 1) * page <= first) for i, p in enumerate(table)), (rc.num_tokens, table)
        held.append(sum(1 for p in table if p >= 0))
        cm.check()
    assert max(held[2:]) <= -(-size // page) + 1 + -(-(2 * size + 1) // page)
    cm.close(rc)
    assert cm.free_pages() == [64]


def test_a_window_group_next_to_blocks_gives_back_by_its_own_rule():
    w = CacheGroupSpec("w", 1, 1, 8, 20, None, 0, False, False)
    assert [w.first_needed(n) for n in (0, 19, 20, 45)] == [0, 0, 1, 26]
    assert CacheGroupSpec("all", 1, 1, 8).first_needed(1000) == 0


def test_the_plain_masks():
    blocks = plain.seen_in_blocks(10, 4)
    assert blocks[5].tolist() == [False] * 4 + [True, True] + [False] * 4 and blocks[4].tolist() == [False] * 4 + [True] + [False] * 5
    assert blocks[3].tolist() == [True] * 4 + [False] * 6
    window = plain.seen_in_window(10, 3)
    assert window[5].tolist() == [False] * 3 + [True] * 3 + [False] * 4 and window[1].tolist() == [True, True] + [False] * 8


def test_the_plain_turns_keep_lengths_and_leave_the_rest():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 12, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 3000])
    for turn in (plain.turn_neighbours, plain.turn_halves):
        y = turn(x, pos, {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0}})
        assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])
        assert torch.allclose(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1))
        # stretched by 4: position 4 p turns as position p does without the stretch
        z = turn(x, pos * 4, {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0}})
        assert torch.allclose(z, turn(x, pos, {"dims": 8, "base": 100.0}))
    a = plain.turn_neighbours(x, pos, {"dims": 8, "base": 100.0})
    b = plain.turn_halves(x[..., [0, 2, 4, 6, 1, 3, 5, 7, 8, 9, 10, 11]], pos, {"dims": 8, "base": 100.0})
    assert torch.allclose(a[..., [0, 2, 4, 6, 1, 3, 5, 7, 8, 9, 10, 11]], b)


def test_the_plain_latent_attention_is_attention_with_the_heads_keys_and_values_written_out():
    """The latent mixer against ordinary attention over the keys and values that its maps give."""
    raw = HEADS64["layers"][1]["mixer"]
    g = torch.Generator().manual_seed(4)
    n, W, H, d, r, dv, R = 70, 64, raw["heads"], raw["dim"], raw["rot_dim"], raw["vdim"], raw["kv_rank"]
    w = {"q": torch.randn(H * (d + r), W, generator=g), "dkv": torch.randn(R + r, W, generator=g), "dkv.norm": torch.rand(R, generator=g) + 0.5,
         "uk": torch.randn(H * d, R, generator=g) * 0.2, "uv": torch.randn(H * dv, R, generator=g) * 0.2, "o": torch.randn(W, H * dv, generator=g)}
    w = {"p." + k: v.double() for k, v in w.items()}
    h = torch.randn(n, W, generator=g, dtype=torch.float64)
    out = plain.latent_attention(raw, w, "p.", h, 1e-6)
    down = h @ w["p.dkv"].T
    c = plain.norm_plain(down[:, :R], w["p.dkv.norm"], 1e-6)
    pos = torch.arange(n)
    t = plain.turn_halves(down[:, R:].view(n, 1, r), pos, raw["rot"]).expand(n, H, r)
    k = torch.cat([(c @ w["p.uk"].T).view(n, H, d), t], dim=-1)
    q = (h @ w["p.q"].T).view(n, H, d + r)
    q = torch.cat([q[..., :d], plain.turn_halves(q[..., d:].contiguous(), pos, raw["rot"])], dim=-1)
    v = (c @ w["p.uv"].T).view(n, H, dv)
    want = plain.softmax_heads(q, k, v, raw["scale"], plain.seen_in_window(n, raw["mask"]["size"])) @ w["p.o"].T
    assert torch.allclose(out, want, atol=1e-9)
