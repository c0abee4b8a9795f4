"""Bobarax without a GPU: configuration, tensor names, what its layers ask of the cache manager, and
the plain implementation's mechanisms on hand-made inputs."""

from __future__ import annotations

import pytest
import torch

import bobarax_configs as bc
import bobarax_plain as plain
from mlx_omnia_b200.cache.manager import CacheManager
from mlx_omnia_b200.config.hydrate import ConfigError
from mlx_omnia_b200.parts.base import KVSpec
from mlx_omnia_b200.parts.model import DecoderModel
from mlx_omnia_b200.registry import resolve_architecture

F64 = torch.float64


def _model(name):
    raw = bc.config(name)
    architecture = resolve_architecture(raw)
    return raw, architecture, DecoderModel(architecture.model_spec(architecture.parse(raw)))


@pytest.mark.parametrize("name", sorted(bc.CONFIGS))
def test_names_and_shapes_match_the_random_checkpoint(name):
    raw, architecture, model = _model(name)
    drawn = bc.tensors(name)
    declared = model.tensors()
    assert {architecture.tensor_name(k) for k in drawn} == set(declared)
    for k, t in drawn.items():
        spec = declared[architecture.tensor_name(k)]
        assert tuple(t.shape) == tuple(spec.shape), k
        assert (spec.kind == "table_i32") == (not t.is_floating_point()), k
    for i, layer in enumerate(raw["layers"]):
        if layer["mixer"].get("kv_from") is not None:
            assert f"l{i}.mix.k" not in drawn and f"l{i}.mix.k.norm" not in drawn and f"l{i}.mix.v" not in drawn
        if layer["mlp"] is None:
            assert f"l{i}.norm2" not in drawn and f"l{i}.norm2b" not in drawn
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            table = drawn[f"l{i}.mlp.table"]
            assert table.shape == (raw["vocab"], layer["mlp"]["router"]["top"])
            assert all(len(set(row)) == len(row) for row in table.tolist())


def test_what_the_layers_ask_of_the_cache():
    _, _, model = _model("K")
    needs = model.cache_needs()
    assert needs[0].kv is None and needs[0].state.shape == (3, 16, 24)  # the recurrence keeps a state, no pages
    assert needs[1].kv == KVSpec(((2, 16), (2, 8)), window=7)  # the owner keeps pages for the wider of two windows
    assert needs[2].kv == KVSpec(((2, 16), (2, 24)), chunk=11) and needs[2].state is None
    assert needs[3].kv is None and needs[3].reads == 1
    assert needs[4].state.shape == (2, 8, 8)
    _, _, model = _model("L")
    needs = model.cache_needs()
    assert needs[1].kv.window == 20 and needs[3].reads == 1 and needs[4].reads == 1


def test_pages_behind_a_run_are_given_back():
    spec = KVSpec(((1, 4), (1, 4)), chunk=10)
    assert [spec.dead_below(n) for n in (0, 9, 10, 19, 20, 25)] == [0, 0, 10, 10, 20, 20]
    both = KVSpec(((1, 4), (1, 4)), window=4, chunk=10)
    assert [both.dead_below(n) for n in (3, 9, 10, 12, 17)] == [0, 6, 10, 10, 14]
    from mlx_omnia_b200.parts.model import CacheNeed

    cache = CacheManager([CacheNeed(spec, None, None)], page_size=4, pages_per_group=8, max_requests=2, allocate=False)
    r = cache.open("r")
    cache.grow(r, 9)
    assert cache.release_behind_window(r) == 0 and r.tables[0] == [0, 1, 2]
    cache.grow(r, 4)  # 13 positions: the run that began at 10 is the only one still readable
    assert cache.release_behind_window(r) == 2 and r.tables[0][:2] == [-1, -1] and r.tables[0][2] >= 0
    cache.grow(r, 12)  # 25 positions: positions below 20 are dead, pages 0 to 4
    cache.release_behind_window(r)
    assert [p >= 0 for p in r.tables[0]] == [False] * 5 + [True] * 2
    cache.close("r")
    cache.check()
    assert cache.groups[0].pool.free == 8


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="mamba"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "divide"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "does not run before"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "none of its kind"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "differ in key/value sizes"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_named_errors(change, message):
    raw = bc.config("K")
    change(raw)
    with pytest.raises(ConfigError, match=message):
        resolve_architecture(raw).parse(raw)


def test_the_plain_recurrence_over_a_cut_and_in_closed_form():
    g = torch.Generator().manual_seed(1)
    T, H, dk, dv = 23, 3, 5, 4
    q, k, v = (torch.randn(T, H, d, generator=g, dtype=F64) for d in (dk, dk, dv))
    decay = [0.5, 0.9, 1.0]
    whole, S = plain.decayed_state_heads(q, k, v, decay)
    first, S1 = plain.decayed_state_heads(q[:9], k[:9], v[:9], decay)
    second, S2 = plain.decayed_state_heads(q[9:], k[9:], v[9:], decay, S1)
    assert torch.allclose(torch.cat([first, second]), whole) and torch.allclose(S2, S)
    # o_t = sum_{j <= t} decay^(t - j) (q_t . k_j) v_j
    t, h = 17, 1
    direct = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
    assert torch.allclose(whole[t, h], direct)


def test_the_plain_masks_and_the_rotation():
    see = plain.sees_chunk(9, 4)
    assert see[5].tolist() == [False, False, False, False, True, True, False, False, False]
    assert see[8].tolist() == [False] * 8 + [True] and see[3].tolist() == [True] * 4 + [False] * 5
    see = plain.sees_window(6, 3)
    assert see[5].tolist() == [False, False, False, True, True, True] and see[1].tolist() == [True, True] + [False] * 4
    x = torch.arange(12, dtype=F64).view(1, 1, 12) + 1
    y = plain.rotate_pairs(x, torch.tensor([3]), 4, 100.0)
    assert torch.equal(y[..., 4:], x[..., 4:])  # dims beyond the rotated ones pass
    for i in range(2):
        a = 3 * 100.0 ** (-2.0 * i / 4)
        u, w = x[0, 0, 2 * i], x[0, 0, 2 * i + 1]
        assert torch.allclose(y[0, 0, 2 * i], u * torch.cos(torch.tensor(a)) - w * torch.sin(torch.tensor(a)))
        assert torch.allclose(y[0, 0, 2 * i + 1], w * torch.cos(torch.tensor(a)) + u * torch.sin(torch.tensor(a)))
    assert torch.allclose(plain.rotate_pairs(x, torch.tensor([0]), 12, 7.0), x)


def test_the_plain_forward_is_causal_and_sees_the_table():
    raw, W = bc.config("K"), bc.tensors("K")
    ids = bc.prompt(30, raw["vocab"], 3)
    full = plain.forward(ids, W, raw)
    assert torch.allclose(plain.forward(ids[:17], W, raw), full[:17], atol=1e-9)
    other = dict(W)
    other["l1.mlp.table"] = (W["l1.mlp.table"] + 1) % 5
    assert (plain.forward(ids, other, raw) - full).abs().max() > 1e-3
