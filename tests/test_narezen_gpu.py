"""Narezen on the GPU against the plain implementation (`narezen_plain`): each mechanism's kernels
alone, then the engine whole, decoded token by token, in portions down to two tokens, in mixed
batches with pages and state slots used again, with keys far away and at page borders, and through
the generation entry point, the command line and the replay program."""

from __future__ import annotations

import subprocess
import sys

import pytest
import torch

import narezen_configs as nc
import narezen_plain as plain
from mlx_omnia_b200 import GenerationOptions, load
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.step import StepEntry
from mlx_omnia_b200.engine.trace import poison_free_pages
from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import KVSpec, KVView
from trace_tools import ROOT, Trace, stacked

pytestmark = pytest.mark.gpu
CUDA = torch.device("cuda:0")
F64 = torch.float64
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rel(a, b) -> float:
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


class Batch:
    """A step's metadata for kernels that are called alone: requests that bring `lens` tokens each
    and held `starts` positions before, in state slots `slots`."""

    def __init__(self, lens, starts=None, slots=None):
        starts = starts or [0] * len(lens)
        self.num_seqs, self.q_lens = len(lens), list(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        self.num_tokens = cu[-1]
        self.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=CUDA)
        self.state_slots = torch.tensor(slots or list(range(len(lens))), dtype=torch.int32, device=CUDA)
        self.positions = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32, device=CUDA)
        self.seq_lens = torch.tensor([s + n for s, n in zip(starts, lens)], dtype=torch.int32, device=CUDA)
        self.seq_lens_host = [s + n for s, n in zip(starts, lens)]
        self.max_q_len, self.max_seq_len, self.workspace = max(lens), max(self.seq_lens_host), None
        self.decode_only = all(n == 1 for n in lens)
        self.token_ids = None


# ---- each mechanism alone -------------------------------------------------------------------


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv,cols,rot,channel", [(3, 16, 24, None, 8, False), (2, 64, 32, 16, 64, True),
                                                      (5, 12, 20, 20, 0, True), (3, 5, 7, None, 4, False),
                                                      (2, 128, 128, 32, 32, True), (1, 32, 16, 4, 32, False),
                                                      (2, 256, 40, None, 0, False), (2, 8, 24, 24, 0, True)])
def test_state_attention_over_portions_and_slots(dtype, H, dk, dv, cols, rot, channel):
    """Two requests in portions of 1 to 37 tokens from state slots that others used before: the state
    carried in float32 gives the plain recurrence over the whole sequence, with a decay per head or per
    token and key channel, rotated or not, a head's columns cut into runs or not (also a last short run);
    then four steps of one token each (the kernel that does a decoding step in one launch)."""
    g = torch.Generator().manual_seed(dk * 3 + dv)
    dt = DTYPES[dtype]
    Ta, Tb = 79, 45
    width = 2 * H * dk + 2 * H * dv
    decay = [0.5, 0.9, 0.97, 0.999, 1.0][:H]
    tau, q_scale, k_scale = 2.5, 0.7, dk ** -0.5
    rows = {r: (torch.randn(T, width + 4, generator=g) * 1.5).to(dt) for r, T in (("a", Ta), ("b", Tb))}
    logits = {r: (torch.randn(T, H * dk + 3, generator=g) * 2.0 + 1.0).to(dt) for r, T in (("a", Ta), ("b", Tb))}
    bias = torch.randn(H * dk, generator=g)
    w = 1.0 + 0.2 * torch.randn(dv, generator=g)
    inv_freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=CUDA) if rot else None
    S = torch.full((5, H, dk, dv), 3.0, dtype=torch.float32, device=CUDA)
    S[[3, 1]] = 0.0
    got = {"a": [], "b": []}
    cuts = {"a": [0, 37, 38, 40, 56, 75, 76, 77, 78, 79], "b": [0, 1, 18, 19, 20, 41, 42, 43, 44, 45]}
    for i in range(9):
        a0, a1, b0, b1 = cuts["a"][i], cuts["a"][i + 1], cuts["b"][i], cuts["b"][i + 1]
        step = Batch([a1 - a0, b1 - b0], [a0, b0], [3, 1])
        proj = torch.cat([rows["a"][a0:a1], rows["b"][b0:b1]]).to(CUDA)
        z = torch.cat([logits["a"][a0:a1], logits["b"][b0:b1]]).to(CUDA)[:, : H * dk] if channel else None
        out = ops.state_attention(proj, 2, 2 + H * dk, 2 + 2 * H * dk, 2 + 2 * H * dk + H * dv, H, dk, dv, S, step, 1e-5,
                                  decay=None if channel else torch.tensor(decay, device=CUDA), decay_logits=z,
                                  decay_bias=bias.to(CUDA) if channel else None, tau=tau, inv_freq=inv_freq,
                                  q_scale=q_scale, k_scale=k_scale, norm_weight=w.to(CUDA) if channel else None,
                                  gate="silu" if channel else "sigmoid", cols=None if step.decode_only else cols)
        got["a"].append(out[: a1 - a0])
        got["b"].append(out[a1 - a0:])
    for r, T in (("a", Ta), ("b", Tb)):
        x = rows[r].to(F64)[:, 2:]
        q, k = (x[:, i * H * dk: (i + 1) * H * dk].view(T, H, dk) for i in (0, 1))
        if rot:
            q, k = (plain.rotate_half(y, torch.arange(T), rot, 50.0) for y in (q, k))
        v = x[:, 2 * H * dk: 2 * H * dk + H * dv].view(T, H, dv)
        if channel:
            a = torch.exp(torch.nn.functional.logsigmoid(logits[r].to(F64)[:, : H * dk] + bias.to(F64)) / tau).view(T, H, dk)
        else:
            a = torch.tensor(decay, dtype=F64)[None, :, None].expand(T, H, dk)
        o, last = plain.decayed_state_heads(q * q_scale, k * k_scale, v, a)
        gate = x[:, 2 * H * dk + H * dv: width]
        want = plain.rms(o, 1e-5, w.to(F64) if channel else None).reshape(T, H * dv)
        want = want * (plain.silu(gate) if channel else torch.sigmoid(gate))
        assert rel(torch.cat(got[r]), want) < (3e-5 if dtype == "float32" else 1e-2), r
        assert rel(S[3 if r == "a" else 1], last) < 3e-5  # the state's inputs are not rounded: float32 in both
    assert float((S[[0, 2, 4]] - 3.0).abs().max()) == 0.0  # nobody else's slot was touched
    ops.raise_on_error(CUDA)


def test_a_far_token_shows_through_a_slow_decay_and_not_through_a_fast_one():
    """One head forgets at 0.5 a token, one keeps everything (a decay of one): 600 tokens later the first
    token's value still is the second head's output, and nothing of it is left in the first head's."""
    H, dk, dv, T = 2, 16, 8, 600
    proj = torch.zeros(T, 2 * H * dk + 2 * H * dv, dtype=torch.float32)
    proj[:, : H * dk] = 1.0  # every query sees every key channel
    proj[0, H * dk: 2 * H * dk] = 1.0  # only the first token writes
    proj[0, 2 * H * dk: 2 * H * dk + H * dv] = torch.arange(1, H * dv + 1, dtype=torch.float32)
    proj[:, 2 * H * dk + H * dv:] = 30.0  # an open sigmoid gate
    S = torch.zeros(1, H, dk, dv, device=CUDA)
    out = []
    for a, b in [(0, 1), (1, 300), (300, 599), (599, 600)]:
        out.append(ops.state_attention(proj[a:b].to(CUDA), 0, H * dk, 2 * H * dk, 2 * H * dk + H * dv, H, dk, dv, S,
                                       Batch([b - a], [a], [0]), 1e-6, decay=torch.tensor([0.5, 1.0], device=CUDA),
                                       norm_weight=None, gate="sigmoid"))
    last = torch.cat(out)[-1].view(H, dv).cpu()
    v = torch.arange(1, H * dv + 1, dtype=torch.float32).view(H, dv)
    assert torch.allclose(last[1], v[1] / v[1].pow(2).mean().sqrt(), rtol=1e-4)
    assert float(S[0, 0].abs().max()) == 0.0 and float(S[0, 1].min()) > 0.0  # 0.5^599 is nothing in float32


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C,blocks,K", [(48, 3, 3), (64, 1, 1), (30, 5, 5), (160, 2, 4), (512, 4, 16)])
def test_gated_channel_recurrence_over_portions_and_slots(dtype, C, blocks, K):
    """Two requests in portions of 1 to 700 tokens (shorter than the convolution's reach, and long
    enough for the scan to be cut into segments) from slots that others used before, then six steps of
    one token each (the kernel that does a decoding step in one launch)."""
    g = torch.Generator().manual_seed(C + K)
    dt = DTYPES[dtype]
    bw = C // blocks
    Ta, Tb = 796, 47
    rows = {r: (torch.randn(T, 2 * C + 3, generator=g)).to(dt) for r, T in (("a", Ta), ("b", Tb))}
    W = {"x.b": torch.randn(C, generator=g) * 0.3, "y.b": torch.randn(C, generator=g) * 0.3,
         "conv": torch.randn(C, K, generator=g) * K ** -0.5, "conv.b": torch.randn(C, generator=g) * 0.1,
         "ra": torch.randn(blocks, bw, bw, generator=g) * bw ** -0.5, "ri": torch.randn(blocks, bw, bw, generator=g) * bw ** -0.5,
         "ra.b": torch.randn(blocks, bw, generator=g), "ri.b": torch.randn(blocks, bw, generator=g),
         "lam": torch.randn(C, generator=g) - 2.0}
    dev = {k: v.to(CUDA) for k, v in W.items()}
    gates = torch.cat([dev["ra"].transpose(1, 2), dev["ri"].transpose(1, 2)], dim=2).contiguous()
    S = torch.full((5, C), 3.0, dtype=torch.float32, device=CUDA)
    conv = torch.full((5, max(K - 1, 1), C), 3.0, dtype=torch.float32, device=CUDA)
    S[[3, 1]] = 0.0
    conv[[3, 1]] = 0.0
    got = {"a": [], "b": []}
    cuts = {"a": [0, 37, 38, 40, 56, 75, 775, 790] + list(range(791, 797)), "b": [0, 1, 2, 3, 19, 20, 21, 41] + list(range(42, 48))}
    for i in range(13):
        a0, a1, b0, b1 = cuts["a"][i], cuts["a"][i + 1], cuts["b"][i], cuts["b"][i + 1]
        step = Batch([a1 - a0, b1 - b0], [a0, b0], [3, 1])
        proj = torch.cat([rows["a"][a0:a1], rows["b"][b0:b1]]).to(CUDA)
        out = ops.gated_channel_recurrence(proj, 1, 1 + C, dev["x.b"], dev["y.b"], dev["conv"], dev["conv.b"], gates,
                                           dev["ra.b"].reshape(-1), dev["ri.b"].reshape(-1), dev["lam"], 8.0, S, conv, step)
        got["a"].append(out[: a1 - a0])
        got["b"].append(out[a1 - a0:])
    eye = torch.eye(C, dtype=F64)
    for r, T in (("a", Ta), ("b", Tb)):
        x = rows[r].to(F64)
        # The plain block with identity projections: h = [x part | y part] picked by 0/1 matrices.
        h = x[:, 1: 1 + 2 * C]
        pick = {"x": torch.cat([eye, torch.zeros(C, C, dtype=F64)], 1), "y": torch.cat([torch.zeros(C, C, dtype=F64), eye], 1),
                "o": eye}
        want = plain.gated_recurrent_unit(h, {**{k: v.to(F64) for k, v in W.items()}, **pick}, "",
                                          {"width": C, "blocks": blocks, "conv": K})
        assert rel(torch.cat(got[r]), want) < (3e-5 if dtype == "float32" else 8e-3), r
    assert float((S[[0, 2, 4]] - 3.0).abs().max()) == 0.0 and float((conv[[0, 2, 4]] - 3.0).abs().max()) == 0.0
    ops.raise_on_error(CUDA)


def _cache(G, dk, dv, page, count, dtype):
    spec = KVSpec(((G, dk), (G, dv)))
    shape = (count, 2, G, page, dk) if dk == dv else (count, (dk + dv) * G * page)
    return spec, torch.full(shape, float("nan"), dtype=dtype, device=CUDA)


def _view(spec, pages, tables, page, slots):
    width = max(len(t) for t in tables)
    table = torch.full((len(tables), width), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
    return KVView(pages, table.to(CUDA), torch.tensor(slots, dtype=torch.int64, device=CUDA), page, None, writes=True, spec=spec)


@pytest.mark.parametrize("dtype,H,G,d,page", [("float32", 4, 2, 16, 4), ("bfloat16", 4, 2, 64, 16), ("bfloat16", 6, 3, 64, 16),
                                              ("bfloat16", 5, 1, 12, 8), ("float32", 2, 1, 32, 16)])
@pytest.mark.parametrize("learned", [True, False])
def test_keys_as_values_attention_with_a_sink_and_a_far_key(dtype, H, G, d, page, learned):
    """A prompt of 700 tokens in shuffled pages, then a portion over it and single tokens: weightless
    head norms, values that are the keys as projected, a sink a head (learned, or the fixed zero). One key
    far back (position 3, and one at a page's last place) is made to stand out for the last queries, so
    that losing it would show; the sink is shown to count."""
    g = torch.Generator().manual_seed(d + H)
    dt = DTYPES[dtype]
    T, eps, scale = 760, 1e-5, 0.9
    proj = (torch.randn(T, (H + G) * d + 8, generator=g) * 1.3).to(dt)
    far = [3, 5 * page - 1]
    for t in far:
        proj[t, H * d: (H + G) * d] *= 6.0  # a loud key (and value: they are the same numbers)
    sink = (torch.randn(H, generator=g) + 1.0) if learned else torch.zeros(H)
    pages_needed = -(-T // page)
    order = torch.randperm(pages_needed + 7, generator=g)[:pages_needed].tolist()
    spec, pages = _cache(G, d, d, page, pages_needed + 7, dt)
    slot_of = lambda t: order[t // page] * page + t % page  # noqa: E731
    got = []
    for a, b in [(0, 700), (700, 741)] + [(t, t + 1) for t in range(741, T)]:
        step = Batch([b - a], [a], [0])
        kv = _view(spec, pages, [order[: -(-b // page)]], page, [slot_of(t) for t in range(a, b)])
        rows = proj[a:b].to(CUDA)
        q = ops.qkv_prepare(rows, 0, H * d, H * d, H, d, None, None, None, eps, None, step.positions, kv, store=True)
        got.append(ops.paged_attention(q, kv, step, scale, sink=sink.to(CUDA)))
    x = proj.to(F64)
    q, k = x[:, : H * d].view(T, H, d), x[:, H * d: (H + G) * d].view(T, G, d)
    qn, kn = (plain.rms(y, eps).to(dt).to(F64) for y in (q, k))  # the kernels round what they keep
    want = plain.sink_softmax_heads(qn, kn, k, scale, sink.to(F64))
    tolerance = 3e-5 if dtype == "float32" else 2e-2
    assert rel(torch.cat(got).view(T, -1), want) < tolerance
    without = plain.sink_softmax_heads(qn, kn, k, scale, torch.full((H,), -1e9, dtype=F64))
    assert rel(without[:16], want[:16]) > 5 * tolerance  # the sink is not a detail (least of all with few keys)
    k_lost = k.clone()
    k_lost[far[0]] = 0.0
    lost = plain.sink_softmax_heads(qn, plain.rms(k_lost, eps), k_lost, scale, sink.to(F64))
    assert rel(lost[700:], want[700:]) > 5 * tolerance  # nor is the far key
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype,tensor_cores,tcgen05", [("float32", False, False), ("bfloat16", True, False),
                                                        ("bfloat16", False, False), ("bfloat16", True, True)])
@pytest.mark.parametrize("rows,hidden,inner,experts,top,shared", [(50, 96, 24, 5, 2, 40), (1, 64, 40, 3, 1, None),
                                                                  (300, 128, 64, 4, 4, 16), (7, 100, 12, 2, 1, 20)])
def test_sigmoid_routed_experts_weighted_on_their_inputs(dtype, tensor_cores, tcgen05, rows, hidden, inner, experts, top, shared):
    if tensor_cores and (hidden % 8 or inner % 8):
        pytest.skip("the tensor-core products take widths in eights")
    g = torch.Generator().manual_seed(rows + hidden)
    dt = DTYPES[dtype]
    W = {"router": torch.randn(experts, hidden, generator=g) * 2.0 * hidden ** -0.5}
    for name, width in [(f"e{e}", inner) for e in range(experts)] + ([("shared", shared)] if shared else []):
        W[f"{name}.gate"], W[f"{name}.up"] = (torch.randn(width, hidden, generator=g) * 2.0 * hidden ** -0.5 for _ in range(2))
        W[f"{name}.down"] = torch.randn(hidden, width, generator=g) * width ** -0.5
    W = {k: (v if k == "router" else v.to(torch.bfloat16).float()) for k, v in W.items()}
    h = torch.randn(rows, hidden, generator=g).to(dt)
    gate_up = torch.stack([torch.cat([W[f"e{e}.gate"], W[f"e{e}.up"]]) for e in range(experts)]).to(dt).to(CUDA)
    down = torch.stack([W[f"e{e}.down"] for e in range(experts)]).to(dt).to(CUDA)
    extra = None
    if shared:
        extra = ops.linear(ops.linear_swiglu(h.to(CUDA), torch.cat([W["shared.gate"], W["shared.up"]]).to(dt).to(CUDA)),
                           W["shared.down"].to(dt).to(CUDA))
    got = ops.moe_experts(h.to(CUDA), W["router"].to(CUDA), None, gate_up, down, top, None, tensor_cores=tensor_cores,
                          tcgen05=tcgen05, scoring="sigmoid", weigh="input", extra=extra)
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.routed_experts(h.to(F64), {k: v.to(F64) for k, v in W.items()}, "", mlp)
    err = (got.cpu().double() - want).abs().amax(-1) / want.abs().max()
    # In bfloat16 a choice between two nearly equal scores may fall the other way: bound the rows, not the row.
    assert float(err.median()) < (2e-5 if dtype == "float32" else 1e-2)
    assert float((err > (2e-5 if dtype == "float32" else 3e-2)).float().mean()) <= (0.0 if dtype == "float32" else 0.03)
    after = plain.routed_experts(h.to(F64), {k: v.to(F64) for k, v in W.items()}, "", {**mlp, "shared": None})
    assert shared is None or rel(after, want) > 1e-2  # the shared expert is not a detail
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_branches_meet_with_a_constant_each(dtype):
    g = torch.Generator().manual_seed(5)
    a, b = (torch.randn(37, 100, generator=g).to(DTYPES[dtype]) for _ in range(2))
    got = ops.scaled_sum(a.to(CUDA), 1.2, b.to(CUDA), -0.5)
    want = (1.2 * a.double() - 0.5 * b.double())
    assert rel(got, want) < (1e-6 if dtype == "float32" else 4e-3)


# ---- the engine -----------------------------------------------------------------------------


def engine_for(name, dtype="float32", page=4, tokens=1024, requests=4, graphs=True, seed=0, raw=None):
    raw = raw or nc.config(name)
    weights = nc.tensors(name if raw == nc.CONFIGS.get(name) else raw, seed)
    engine = Engine.from_tensors(raw, weights, EngineArgs(dtype=dtype, page_size=page, cache_tokens=tokens,
                                                          max_requests=requests, cuda_graphs=graphs))
    return raw, weights, engine


TOLERANCE = {"float32": 3e-4, "bfloat16": 8e-2}


def every_expert(raw) -> bool:
    """Whether every token uses every expert of every layer (no choice that rounding could turn)."""
    return all(l["mlp"] is None or l["mlp"]["router"]["top"] == l["mlp"]["router"]["experts"] for l in raw["layers"])


def assert_rows(got, want, dtype, what="", tolerance=None, strict=False):
    """Rows of logits against rows of the plain implementation. float32: every row within the tolerance
    (of the largest logit). bfloat16: the median row within a third of it and at most one row in ten
    beyond it: a routed layer's choice between two nearly equal scores can fall the other way than in
    float64, which moves that row by tens of per cent and, through the states and the cache, the rows
    after it by a little; with these configurations' few experts that happens to a few rows in a hundred.
    `strict` (a configuration without such choices): every row within the tolerance in bfloat16 too."""
    tolerance = tolerance or TOLERANCE[dtype]
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    assert got.shape == want.shape
    err = (got - want).abs().amax(-1) / want.abs().max().clamp_min(1e-30)
    assert not torch.isnan(err).any(), what
    if dtype == "float32" or strict:
        assert float(err.max()) < tolerance, (what, int(err.argmax()), float(err.max()))
    else:
        assert float(err.median()) < tolerance / 3, (what, float(err.median()))
        assert int((err >= tolerance).sum()) <= max(3, len(err) // 10), (what, err.topk(min(5, len(err))))


@pytest.mark.parametrize("name", sorted(nc.CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(name, dtype):
    raw, weights, engine = engine_for(name, dtype)
    for n in (1, 2, 3, 41, 230):
        ids = nc.prompt(n, raw["vocab"], n)
        request = engine.cache.open("r")
        got = engine.runner.run([StepEntry(request, ids, list(range(n)))])
        engine.cache.close("r")
        assert_rows(got, plain.forward(ids, weights, raw), dtype, n, strict=every_expert(raw))
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("name,page", [("P", 4), ("Q", 16), ("R", 8)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_decoding_and_mixed_batches(tmp_path, name, page, dtype):
    """Six requests over four state slots: prompts read whole, in portions of 2 to 9 tokens and
    token by token, decoded tokens beside portions of other requests, requests that end and whose
    pages and slots the next ones take (free pages are filled with NaN before every step)."""
    raw, weights, engine = engine_for(name, dtype, page=page, tokens=448)
    V = raw["vocab"]
    ids = {r: nc.prompt(n, V, i) for i, (r, n) in enumerate({"a": 170, "b": 33, "c": 2, "d": 58, "e": 60, "f": 17}.items())}
    trace = Trace()
    at = {r: 0 for r in ids}

    def take(r, n):
        out = ids[r][at[r]: at[r] + n]
        at[r] += len(out)
        return out

    trace.step({"a": take("a", 9), "b": take("b", 33)})
    trace.step({"a": take("a", 2), "c": take("c", 1), "d": take("d", 5)}, end=["b"])
    trace.step({"a": take("a", 7), "c": take("c", 1), "d": take("d", 3), "e": take("e", 40)}, end=["c"])
    for _ in range(6):
        trace.step({"a": take("a", 1), "d": take("d", 2), "e": take("e", 1)})
    trace.step({"f": take("f", 17), "a": take("a", 1)}, end=["f"])
    for _ in range(3):
        trace.step({"e": take("e", 1), "a": take("a", 4), "d": take("d", 1)})
    trace.step({"a": take("a", 97)})
    for _ in range(12):
        trace.step({"a": take("a", 1), "d": take("d", 1)})
    trace.step({"a": take("a", 170), "d": take("d", 58), "e": take("e", 60)}, end=["a", "d", "e"])
    got = trace.run_engine(engine, tmp_path / "out", before_step=lambda e, record: poison_free_pages(e))
    assert not engine.cache.requests
    engine.cache.check()
    for r in ids:
        positions, logits = stacked(got[r])
        assert positions == list(range(len(ids[r])))
        assert_rows(logits, plain.forward(ids[r], weights, raw), dtype, r, strict=every_expert(raw))


@pytest.mark.parametrize("name", sorted(nc.CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_decoding_token_by_token(name, dtype):
    """The same prompt whole, and one token a step (captured decode steps, and launched one by one)."""
    for graphs in (True, False):
        raw, weights, engine = engine_for(name, dtype, graphs=graphs)
        ids = nc.prompt(75, raw["vocab"], 77)
        request = engine.cache.open("w")
        whole = engine.runner.run([StepEntry(request, ids, list(range(len(ids))))])
        engine.cache.close("w")
        request = engine.cache.open("t")
        single = torch.cat([engine.runner.run([StepEntry(request, [t], [0])]) for t in ids])
        engine.cache.close("t")
        assert_rows(single, whole, dtype, "token by token against whole", 3e-5 if dtype == "float32" else 6e-2,
                    strict=every_expert(raw))
        assert_rows(single, plain.forward(ids, weights, raw), dtype, strict=every_expert(raw))
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_across_tiles_chunks_and_pages(dtype):
    """700 tokens with slow decays: portions that start and end inside tiles of 64 keys, decode chunks of
    128 and pages of 16, the last token a repeat of an early one, then 40 tokens decoded beside a short
    request whose pages are the ones nobody held before."""
    raw, weights, engine = engine_for("Q", dtype, page=16, tokens=1024)
    ids = nc.prompt(700, raw["vocab"], 5)
    ids[-1] = ids[11]
    other = nc.prompt(50, raw["vocab"], 6)
    a = engine.cache.open("a")
    rows = {}
    at = 0
    for n in (193, 2, 130, 61, 255, 19):
        out = engine.runner.run([StepEntry(a, ids[at: at + n], [n - 1])])
        rows[at + n - 1] = out[0]
        at += n
    b = engine.cache.open("b")
    engine.runner.run([StepEntry(b, other[:10], [])])
    for t in range(at, 700):
        out = engine.runner.run([StepEntry(a, ids[t: t + 1], [0]), StepEntry(b, other[10 + t - at: 11 + t - at], [0])])
        rows[t] = out[0]
        rows[("b", 10 + t - at)] = out[1]
    expect, expect_b = plain.forward(ids, weights, raw), plain.forward(other, weights, raw)
    keys = list(rows)
    assert_rows(torch.stack([rows[key] for key in keys]),
                torch.stack([expect_b[key[1]] if isinstance(key, tuple) else expect[key] for key in keys]), dtype, keys,
                strict=True)
    ops.raise_on_error(CUDA)


def test_the_constants_show_in_the_logits():
    """A decay, a tau, a branch's constant, a rotation's width or base, the attention's scale, the
    experts a token uses or the embedding's scale moved a little: each moves the plain implementation's
    logits by far more than the engine is from it, so the comparisons above see such a fault. In a prompt
    and in decoding."""
    raw, weights, engine = engine_for("P", "float32")
    ids = nc.prompt(48, raw["vocab"], 8)
    request = engine.cache.open("r")
    got = [engine.runner.run([StepEntry(request, ids[:30], list(range(30)))])]
    got += [engine.runner.run([StepEntry(request, [t], [0])]) for t in ids[30:]]
    expect = plain.forward(ids, weights, raw)
    assert rel(torch.cat(got), expect) < TOLERANCE["float32"]

    def moved(change):
        other = nc.config("P")
        change(other)
        out = plain.forward(ids, weights, other)
        return min(rel(out[:30], expect[:30]), rel(out[30:], expect[30:]))

    assert moved(lambda c: c["layers"][1]["mixer"]["right"]["decay"].__setitem__(2, 0.9)) > 1e-3
    assert moved(lambda c: c["layers"][2]["mixer"]["right"].update(tau=4.0)) > 1e-3
    assert moved(lambda c: c["layers"][2]["mixer"].update(left_scale=1.0)) > 1e-3
    assert moved(lambda c: c["layers"][1]["mixer"].update(right_scale=1.2)) > 1e-3
    assert moved(lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=6)) > 1e-3
    assert moved(lambda c: c["layers"][1]["mixer"]["right"]["rot"].update(base=60.0)) > 1e-3
    assert moved(lambda c: c["layers"][3]["mixer"]["left"].update(scale=0.5)) > 1e-3
    assert moved(lambda c: c["layers"][0]["mlp"]["router"].update(top=1)) > 1e-3
    assert moved(lambda c: c["embedding"].update(scale=1.4)) > 1e-3
    assert moved(lambda c: c.update(logit_softcap=10.0)) > 1e-3


def test_greedy_generation_long_decoding_and_the_scheduler(tmp_path):
    """Through `load(...).generate`: the scheduler admits, batches and chunks; greedy ids are the plain
    implementation's best, 200 tokens past a two-token prompt included (the states are carried through
    all of them)."""
    raw = nc.config("P")
    weights = nc.tensors("P", 3)
    folder = tmp_path / "m"
    nc.write_folder(folder, raw, weights)
    model = load(folder, dtype="float32", page_size=8, cache_tokens=1024, max_requests=4, max_tokens_per_step=16)
    prompts = [nc.prompt(n, raw["vocab"], 20 + n) for n in (2, 5, 23, 40, 9, 31)]
    counts = [200, 12, 12, 12, 12, 12]
    got = [model.generate([prompts[0]], GenerationOptions(max_tokens=200, stop=()))[0]]
    got += model.generate(prompts[1:], GenerationOptions(max_tokens=12, stop=()))
    for prompt, ids, count in zip(prompts, got, counts):
        assert len(ids) == count
        logits = plain.forward(prompt + ids, weights, raw)[len(prompt) - 1: -1]
        best = logits.max(dim=-1).values
        chosen = logits[torch.arange(count), torch.tensor(ids)]
        assert float((best - chosen).max()) <= 1e-3 * float(logits.abs().max())
    assert not model.engine.cache.requests
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "omnia"), "run", "-m", str(folder), "--max-tokens", "5",
                           "--temperature", "0", "--dtype", "float32", *map(str, prompts[1])],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    assert [int(t) for t in done.stdout.split()[:5]] == got[1][:5]


def test_replay_program_on_a_model_folder(tmp_path):
    """`bin/trace_run` as a user runs it, in bfloat16, on a folder written by the random-weights mode."""
    from safetensors.torch import load_file

    from mlx_omnia_b200.weights.random_init import write_random_model

    raw = nc.config("Q")
    folder = write_random_model(tmp_path / "m", raw, seed=4)
    weights = {k: v.float() for k, v in load_file(str(folder / "model.safetensors")).items()}
    ids = nc.prompt(90, raw["vocab"], 1)
    trace = Trace()
    trace.step({"p": ids[:50]}, want="last")
    trace.step({"p": ids[50:52], "q": ids[:7]})
    for t in range(52, 90):
        trace.step({"p": ids[t: t + 1]}, end=["p"] if t == 89 else ["q"] if t == 52 else [])
    got = trace.run(folder, "bfloat16", tmp_path / "out", vocab=raw["vocab"])
    expect = plain.forward(ids, weights, raw)
    positions, logits = stacked(got["p"])
    assert positions == [49] + list(range(50, 90))
    assert_rows(logits, expect[positions], "bfloat16", strict=True)
