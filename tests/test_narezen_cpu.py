"""Narezen without a GPU: configuration, tensor names, what its layers ask of the cache manager, and
the plain implementation's mechanisms on hand-made inputs."""

from __future__ import annotations

import math

import pytest
import torch

import narezen_configs as nc
import narezen_plain as plain
from mlx_omnia_b200.config.hydrate import ConfigError
from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import KVSpec, PartSpec
from mlx_omnia_b200.parts.model import DecoderModel
from mlx_omnia_b200.parts.recurrent import SideBySide
from mlx_omnia_b200.registry import resolve_architecture

F64 = torch.float64


def _model(name, rank=None):
    raw = nc.config(name)
    architecture = resolve_architecture(raw)
    drawn = nc.tensors(name, rank=rank)
    config = architecture.sizes_from_tensors(architecture.parse(raw), lambda n: tuple(drawn[n].shape) if n in drawn else None)
    return raw, architecture, drawn, DecoderModel(architecture.model_spec(config))


@pytest.mark.parametrize("name", sorted(nc.CONFIGS))
def test_names_and_shapes_match_the_random_checkpoint(name):
    raw, architecture, drawn, model = _model(name)
    declared = model.tensors()
    assert {architecture.tensor_name(k) for k in drawn} == set(declared)
    for k, t in drawn.items():
        assert tuple(t.shape) == tuple(declared[architecture.tensor_name(k)].shape), k
    for i, layer in enumerate(raw["layers"]):
        if layer["mlp"] is None:
            assert f"l{i}.norm2" not in drawn and f"l{i}.mlp.router" not in drawn
        else:
            assert (f"l{i}.mlp.shared.gate" in drawn) == ("shared" in layer["mlp"])
        if layer["type"] == "parallel":
            assert f"l{i}.mix.left.v" not in drawn and f"l{i}.mix.left.sink" in drawn
            assert drawn[f"l{i}.mix.right.a1"].shape[0] == nc.DECAY_RANKS[name]
        if layer["type"] == "parallel_2":
            assert f"l{i}.mix.left.sink" not in drawn and f"l{i}.mix.right.norm" not in drawn


def test_the_decay_maps_inner_width_comes_from_the_tensors():
    for rank in (1, 7):
        _, _, drawn, model = _model("P", rank=rank)
        assert model.tensors()["l2.mix.right.a2"].shape == (2 * 8, rank)


def test_what_the_layers_ask_of_the_cache():
    _, _, _, model = _model("P")
    needs = model.cache_needs()
    assert needs[0].kv is None and set(needs[0].state) == {"S", "conv"}
    assert needs[0].state["S"].shape == (48,) and needs[0].state["conv"].shape == (2, 48)
    assert needs[1].kv == KVSpec(((2, 16), (2, 24))) and needs[1].state.shape == (3, 16, 8)
    assert needs[2].kv == KVSpec(((2, 16), (2, 16))) and needs[2].state.shape == (2, 8, 24)
    assert all(need.reads is None for need in needs)
    _, _, _, model = _model("Q")
    assert model.cache_needs()[1].state["conv"].shape == (1, 64)  # a single tap keeps no inputs; the slot has a row


def test_two_stateful_sides_keep_their_state_apart():
    one = PartSpec("gated_state_attention", {"hidden": 16, "heads": 2, "dim": 4, "vdim": 4, "norm_eps": 1e-5,
                                             "decay": (0.5, 0.9)})
    two = PartSpec("gated_channel_recurrence", {"hidden": 16, "width": 8, "blocks": 2, "conv": 3})
    both = SideBySide(one, two, 1.0, 2.0)
    assert set(both.state_spec()) == {"left", "right.S", "right.conv"} and both.kv_spec() is None
    state = {"left": 1, "right.S": 2, "right.conv": 3}
    assert both._state_of("left", state) == 1 and both._state_of("right", state) == {"S": 2, "conv": 3}
    attention = PartSpec("sink_window_attention", {"hidden": 16, "heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 1.0})
    with pytest.raises(ValueError):
        SideBySide(attention, attention)


def test_named_errors():
    def broken(change):
        raw = nc.config("P")
        change(raw)
        return raw

    architecture = resolve_architecture(nc.config("P"))
    for change, word in [(lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "decay"),
                         (lambda c: c["layers"][2]["mixer"]["left"].update(vdim=8), "keys"),
                         (lambda c: c["layers"][2]["mixer"]["right"].pop("tau"), "tau"),
                         (lambda c: c["layers"][0]["mixer"].update(blocks=5), "blocks"),
                         (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18), "rot"),
                         (lambda c: c["layers"][3]["mlp"]["router"].update(top=4), "experts"),
                         (lambda c: c["layers"][0].update(type="other"), "unknown type"),
                         (lambda c: c.pop("vocab"), "vocab")]:
        with pytest.raises(ConfigError, match=word):
            architecture.parse(broken(change))


def test_the_plain_recurrence_over_a_cut_and_in_closed_form():
    g = torch.Generator().manual_seed(1)
    T, H, dk, dv = 23, 2, 3, 4
    q, k, v = (torch.randn(T, H, d, generator=g, dtype=F64) for d in (dk, dk, dv))
    decay = torch.rand(T, H, dk, generator=g, dtype=F64)
    whole, last = plain.decayed_state_heads(q, k, v, decay)
    first, S = plain.decayed_state_heads(q[:9], k[:9], v[:9], decay[:9])
    second, S2 = plain.decayed_state_heads(q[9:], k[9:], v[9:], decay[9:], S)
    assert torch.allclose(torch.cat([first, second]), whole) and torch.allclose(S2, last)
    # o_t = sum_j (q_t * prod_{j < i <= t} a_i) . k_j  v_j
    t, h = 11, 1
    want = torch.zeros(dv, dtype=F64)
    for j in range(t + 1):
        want += ((q[t, h] * decay[j + 1: t + 1, h].prod(0)) @ k[j, h]) * v[j, h]
    assert torch.allclose(whole[t, h], want)


def test_the_plain_sink_counts_once_and_has_no_value():
    g = torch.Generator().manual_seed(2)
    T, dk = 5, 4
    q, k, v = (torch.randn(T, 1, dk, generator=g, dtype=F64) for _ in range(3))
    sink = torch.tensor([0.7], dtype=F64)
    out = plain.sink_softmax_heads(q, k, v, 0.5, sink)
    t = 3
    s = (q[t, 0] @ k[: t + 1, 0].T) * 0.5
    want = (torch.exp(s) @ v[: t + 1, 0]) / (torch.exp(s).sum() + math.exp(0.7))
    assert torch.allclose(out[t], want)
    none = plain.sink_softmax_heads(q, k, v, 0.5, torch.tensor([-1e9], dtype=F64))
    assert torch.allclose(none[0], v[0, 0])  # without a sink the first token returns its own value


def test_the_plain_rotation_pairs_halves_and_passes_the_rest():
    x = torch.arange(12, dtype=F64).view(1, 1, 12) + 1.0
    out = plain.rotate_half(x.expand(3, 1, 12), torch.arange(3), 4, 100.0)
    assert torch.equal(out[0], x[0]) and torch.equal(out[:, :, 4:], x.expand(3, 1, 12)[:, :, 4:])
    a0, a1 = 2.0, 2.0 * 100.0 ** (-2.0 / 4)
    assert torch.allclose(out[2, 0, 0], x[0, 0, 0] * math.cos(a0) - x[0, 0, 2] * math.sin(a0))
    assert torch.allclose(out[2, 0, 3], x[0, 0, 3] * math.cos(a1) + x[0, 0, 1] * math.sin(a1))


def test_the_plain_convolution_and_gated_recurrence():
    g = torch.Generator().manual_seed(3)
    x, taps, bias = torch.randn(6, 2, generator=g, dtype=F64), torch.randn(2, 3, generator=g, dtype=F64), torch.randn(2, dtype=F64, generator=g)
    y = plain.causal_conv(x, taps, bias)
    assert torch.allclose(y[0], bias + taps[:, 2] * x[0])
    assert torch.allclose(y[4], bias + taps[:, 2] * x[4] + taps[:, 1] * x[3] + taps[:, 0] * x[2])
    # One channel, one block, by hand.
    W = {"y": torch.tensor([[0.3]]), "y.b": torch.tensor([0.1]), "x": torch.tensor([[1.0]]), "x.b": torch.tensor([0.2]),
         "conv": torch.tensor([[0.5, 2.0]]), "conv.b": torch.tensor([0.0]), "ra": torch.tensor([[[0.7]]]),
         "ra.b": torch.tensor([[0.1]]), "ri": torch.tensor([[[-0.4]]]), "ri.b": torch.tensor([[0.3]]),
         "lam": torch.tensor([0.5]), "o": torch.tensor([[1.0]])}
    W = {k: v.to(F64) for k, v in W.items()}
    h = torch.tensor([[1.0], [-2.0], [0.5]], dtype=F64)
    got = plain.gated_recurrent_unit(h, W, "", {"width": 1, "blocks": 1, "conv": 2})
    S, before, want = 0.0, 0.0, []
    for t in range(3):
        x_t = float(h[t]) + 0.2
        u = 2.0 * x_t + 0.5 * before
        before = x_t
        r, i = 1 / (1 + math.exp(-(0.7 * u + 0.1))), 1 / (1 + math.exp(-(-0.4 * u + 0.3)))
        a = math.exp(-8.0 * r * math.log1p(math.exp(0.5)))
        S = a * S + math.sqrt(1 - a * a) * i * u
        z = 0.3 * float(h[t]) + 0.1
        want.append(S * 0.5 * z * (1 + math.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))
    assert torch.allclose(got[:, 0], torch.tensor(want, dtype=F64))


def test_the_plain_experts_weigh_their_inputs():
    raw = nc.config("P")
    W = {k: v.to(F64) for k, v in nc.tensors("P").items()}
    g = torch.Generator().manual_seed(4)
    h = torch.randn(9, raw["width"], generator=g, dtype=F64)
    mlp = raw["layers"][0]["mlp"]
    chosen = []
    out = plain.routed_experts(h, W, "l0.mlp.", mlp, chosen)
    scores = torch.sigmoid(h @ W["l0.mlp.router"].T)
    t = 5
    want = plain.gated_expert(h[t: t + 1], W, "l0.mlp.shared.")
    assert len(set(chosen[0][t].tolist())) == 2 and set(chosen[0][t].tolist()) == set(scores[t].topk(2).indices.tolist())
    for e in chosen[0][t].tolist():
        want = want + plain.gated_expert(h[t: t + 1] * scores[t, e], W, f"l0.mlp.e{e}.")
    assert torch.allclose(out[t], want[0])
    weighed_after = sum(scores[t, e] * plain.gated_expert(h[t: t + 1], W, f"l0.mlp.e{e}.") for e in chosen[0][t].tolist())
    assert not torch.allclose(want - plain.gated_expert(h[t: t + 1], W, "l0.mlp.shared."), weighed_after, rtol=1e-3)


@pytest.mark.parametrize("name", sorted(nc.CONFIGS))
def test_the_plain_model_is_causal_and_every_layer_counts(name):
    raw = nc.config(name)
    W = nc.tensors(name)
    ids = nc.prompt(20, raw["vocab"], 1)
    other = list(ids)
    other[13] = (other[13] + 1) % raw["vocab"]
    a, b = plain.forward(ids, W, raw), plain.forward(other, W, raw)
    assert torch.allclose(a[:13], b[:13], rtol=0, atol=1e-11) and not torch.allclose(a[13:], b[13:])
    layers = []
    plain.forward(ids, W, raw, layers_out=layers)
    assert len(layers) == len(raw["layers"])
    assert all(not torch.allclose(x, y) for x, y in zip(layers, layers[1:]))


def test_how_many_columns_a_block_of_the_recurrence_takes():
    for requests, heads, dk, dv in [(1, 2, 32, 64), (8, 16, 128, 128), (1, 1, 256, 512), (3, 3, 5, 7), (64, 8, 64, 96),
                                    (1, 4, 16, 1000)]:
        cols = ops.state_columns(requests, heads, dk, dv, 148)
        threads = 1
        while -(-dk // threads) > 32:
            threads *= 2
        assert 1 <= cols <= min(dv, 96) and cols * threads <= 448
        assert dv % 4 or cols % 4 == 0
    assert ops.state_columns(1, 2, 32, 64, 148) < ops.state_columns(64, 2, 32, 64, 148)  # few requests: more blocks
