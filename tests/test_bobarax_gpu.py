"""Bobarax on the GPU against the plain implementation (`bobarax_plain`): each mechanism's kernels
alone, then the engine whole, decoded token by token, in portions down to two tokens, in mixed
batches with pages and state slots used again, with keys far away, at page borders and at the edges
of the windows and of the runs, and through the generation entry point, the command line and the
replay program."""

from __future__ import annotations

import math
import subprocess
import sys

import pytest
import torch

import bobarax_configs as bc
import bobarax_plain as plain
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

    def __init__(self, lens, starts=None, slots=None, tokens=None):
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
        self.token_ids = None if tokens is None else torch.tensor(tokens, dtype=torch.int32, device=CUDA)


# ---- each mechanism alone -------------------------------------------------------------------


def _cache(G, dk, dv, page, count, dtype, window=None, chunk=None):
    spec = KVSpec(((G, dk), (G, dv)), window, chunk=chunk)
    shape = (count, 2, G, page, dk) if dk == dv else (count, (dk + dv) * G * page)
    return spec, torch.full(shape, float("nan"), dtype=dtype, device=CUDA)


def _view(spec, pages, tables, page, slots=None, writes=True):
    width = max(len(t) for t in tables)
    table = torch.full((len(tables), width), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
    slot_mapping = torch.tensor(slots if slots is not None else [0], dtype=torch.int64, device=CUDA)
    return KVView(pages, table.to(CUDA), slot_mapping, page, spec.window, writes=writes, spec=spec)


@pytest.mark.parametrize("dtype,H,G,dk,dv,rot", [("float32", 4, 2, 16, 24, 8), ("bfloat16", 5, 1, 40, 40, 40),
                                                  ("bfloat16", 3, 3, 24, 8, 0), ("float32", 2, 1, 64, 64, 32),
                                                  ("float32", 3, 3, 20, 12, 4)])
def test_whole_projection_norm_interleaved_rotation_and_cache_write(dtype, H, G, dk, dv, rot):
    """The step between the input projection and the attention: one root mean square over all query
    heads (and one over all key heads) with weights of the projection's size, neighbouring dims
    turned together over part of the head, keys and values of unequal width into shuffled pages."""
    g = torch.Generator().manual_seed(H * 10 + dk)
    T, page, dt = 13, 4, DTYPES[dtype]
    cols = H * dk + G * dk + G * dv
    proj = torch.randn(T, cols + 3, generator=g).to(dt)
    wq, wk = torch.randn(H * dk, generator=g), torch.randn(G * dk, generator=g)
    positions = torch.arange(40, 40 + T)
    inv = torch.tensor([300.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    spec, pages = _cache(G, dk, dv, page, 8, dt)
    order = [5, 2, 7, 0]
    slots = [order[j // page] * page + j % page for j in range(T)]
    kv = _view(spec, pages, [order], page, slots)
    step = Batch([T], [40])
    q = ops.qkv_prepare(proj.to(CUDA), 0, H * dk, H * dk + G * dk, H, dk, None, wq.to(CUDA), wk.to(CUDA), 1e-5,
                        None if inv is None else inv.to(CUDA), step.positions, kv, store=True, whole=True, interleaved=True)
    full = proj.to(F64)
    want_q = plain.whole_projection_norm(full[:, : H * dk], wq, 1e-5).view(T, H, dk)
    want_k = plain.whole_projection_norm(full[:, H * dk: H * dk + G * dk], wk, 1e-5).view(T, G, dk)
    if rot:
        want_q, want_k = (plain.rotate_pairs(x, positions, rot, 300.0) for x in (want_q, want_k))
    want_v = full[:, H * dk + G * dk: cols].view(T, G, dv)
    tolerance = 1e-5 if dtype == "float32" else 1.2e-2
    assert rel(q, want_q) < tolerance
    for j in range(T):
        got_k = kv.row(0)[order[j // page], :, j % page]
        got_v = kv.row(1)[order[j // page], :, j % page]
        assert rel(got_k, want_k[j]) < tolerance and rel(got_v, want_v[j]) < tolerance
    ops.raise_on_error(CUDA)


def _attention_reference(q, K, V, positions, window, chunk, scale, softcap, gate=None):
    """q [T, H, dk] at `positions` over all keys K [N, G, dk], V [N, G, dv]."""
    T, H, dk = q.shape
    G, dv = K.shape[1], V.shape[2]
    out = torch.zeros(T, H, dv, dtype=F64)
    j = torch.arange(K.shape[0])
    for t in range(T):
        i = int(positions[t])
        see = j <= i
        if window:
            see &= i - j < window
        if chunk:
            see &= j // chunk == i // chunk
        for h in range(H):
            s = (K[:, h // (H // G)] @ q[t, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            out[t, h] = torch.softmax(s.masked_fill(~see, -math.inf), 0) @ V[:, h // (H // G)]
    out = out.reshape(T, H * dv)
    return out if gate is None else out * torch.sigmoid(gate)


def _filled(spec, pages, K, V, page, order):
    """Write K, V (position j at page order[j // page]) into the pages through row views."""
    view = _view(spec, pages, [order], page)
    for j in range(K.shape[0]):
        view.row(0)[order[j // page], :, j % page] = K[j].to(pages.dtype).to(CUDA)
        view.row(1)[order[j // page], :, j % page] = V[j].to(pages.dtype).to(CUDA)
    return view


ATTENTION_CASES = [("float32", 4, 2, 16, 24, 4), ("bfloat16", 6, 1, 16, 16, 8), ("bfloat16", 4, 2, 64, 64, 16),
                   ("bfloat16", 2, 2, 32, 8, 16), ("float32", 4, 1, 24, 24, 16), ("bfloat16", 3, 1, 128, 128, 32)]


@pytest.mark.parametrize("dtype,H,G,dk,dv,page", ATTENTION_CASES)
@pytest.mark.parametrize("window,chunk,softcap", [(None, 11, 5.0), (None, 64, None), (None, 130, 30.0), (9, None, None),
                                                  (150, None, None), (None, 1, 2.0), (1, None, None), (None, None, 4.0)])
def test_attention_with_windows_runs_capped_scores_and_a_gate(dtype, H, G, dk, dv, page, window, chunk, softcap):
    """A prompt whole, a portion over a context, single tokens, and all of them in one batch; windows
    and runs that end inside tiles, decode chunks and pages; pages behind them missing from the table."""
    g = torch.Generator().manual_seed(dk + (window or 0) + (chunk or 0))
    dt, N = DTYPES[dtype], 300
    K, V = torch.randn(N, G, dk, generator=g), torch.randn(N, G, dv, generator=g)
    K, V = K.to(dt).to(F64), V.to(dt).to(F64)
    spec, pages = _cache(G, dk, dv, page, 2 * (-(-N // page)) + 3, dt, window, chunk)
    order = torch.randperm(pages.shape[0], generator=g).tolist()[: -(-N // page)]
    kv = _filled(spec, pages, K, V, page, order)
    tolerance = 2e-5 if dtype == "float32" else 2e-2
    for lens, starts in [([N], [0]), ([37], [N - 37]), ([1], [N - 1]), ([1, 1, 1], [N - 1, 140, 63]),
                         ([2, 1, 60, 1], [128, 199, 70, 0])]:
        step = Batch(lens, starts)
        T = sum(lens)
        q = torch.randn(T, H, dk, generator=g).to(dt)
        gate = torch.randn(T, H * dv + 5, generator=g).to(dt)
        tables = []
        for n, s in zip(lens, starts):
            table = list(order[: -(-(s + n) // page)])
            dead = spec.dead_below(s)  # what a request has given back ahead of its first query of the step
            for index in range(dead // page):
                table[index] = -1
            tables.append(table)
        view = _view(spec, pages, tables, page)
        got = ops.paged_attention(q.to(CUDA), view, step, 0.3, gate=gate.to(CUDA), gate_col=5, window=window,
                                  chunk=chunk, softcap=softcap)
        want = _attention_reference(q.to(F64), K, V, step.positions.cpu(), window, chunk, 0.3, softcap,
                                    gate[:, 5:].to(F64))
        assert rel(got, want) < tolerance, (lens, starts)
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype,H,G,dk,dv,page", ATTENTION_CASES)
def test_a_boosted_key_just_inside_and_just_outside(dtype, H, G, dk, dv, page):
    """One key among hundreds is made to stand out (its score is far above all others); the value it
    carries shows in the output exactly when it is inside the window or the run: at their edges, far
    back, in a prompt and in single tokens."""
    g = torch.Generator().manual_seed(7)
    dt, N = DTYPES[dtype], 420
    for window, chunk, query, key, inside in [(100, None, 400, 301, True), (100, None, 400, 300, False),
                                              (None, 112, 400, 336, True), (None, 112, 400, 335, False),
                                              (None, 112, 335, 224, True), (None, None, 419, 3, True),
                                              (257, None, 300, 44, True), (257, None, 300, 43, False)]:
        K, V = torch.randn(N, G, dk, generator=g) * 0.1, torch.randn(N, G, dv, generator=g)
        direction = torch.randn(dk, generator=g)
        direction = direction / direction.norm()
        K[key] = direction * 6.0
        V[key] = 50.0
        K, V = K.to(dt).to(F64), V.to(dt).to(F64)
        spec, pages = _cache(G, dk, dv, page, -(-N // page), dt, window, chunk)
        kv = _filled(spec, pages, K, V, page, list(range(-(-N // page))))
        for lens, starts, row in [([query + 1], [0], query), ([1], [query], 0), ([30, 1], [query - 29, 17], 29)]:
            step = Batch(lens, starts)
            q = (direction * 6.0).repeat(sum(lens), H, 1).to(dt)
            tables = [list(range(-(-(s + n) // page))) for n, s in zip(lens, starts)]
            got = ops.paged_attention(q.to(CUDA), _view(spec, pages, tables, page), step, 1.0, window=window, chunk=chunk)
            want = _attention_reference(q.to(F64), K, V, step.positions.cpu(), window, chunk, 1.0, None)
            assert rel(got, want) < (2e-5 if dtype == "float32" else 2e-2)
            assert (float(got[row].float().mean()) > 40.0) == inside, (window, chunk, query, key, lens)
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("H,G,d,run,softcap", [(4, 1, 128, 1024, 20.0), (2, 2, 64, 960, None), (8, 2, 64, 2048, 3.0)])
def test_long_runs_in_portions_whose_blocks_are_cut_into_parts(H, G, d, run, softcap):
    """A portion of a prompt deep inside a long run: few blocks, each over many key tiles, which the
    prefill kernel cuts into parts that are merged by the last to finish. The run's first key is
    boosted for one query head, so a part that starts a tile late, or a merge that drops the first
    part, shows; the key just ahead of the run is boosted as much and must not show."""
    g = torch.Generator().manual_seed(run + d)
    N, page, dt = 2100, 16, torch.bfloat16
    K, V = torch.randn(N, G, d, generator=g) * 0.3, torch.randn(N, G, d, generator=g)
    direction = torch.randn(d, generator=g)
    direction = direction / direction.norm()
    start = (N - 1) // run * run  # the last run's first position
    K[start], V[start] = direction * 8.0, 30.0
    K[start - 1], V[start - 1] = direction * 8.0, -30.0
    K, V = K.to(dt).to(F64), V.to(dt).to(F64)
    spec, pages = _cache(G, d, d, page, -(-N // page) + 2, dt, None, run)
    order = torch.randperm(pages.shape[0], generator=g).tolist()[: -(-N // page)]
    kv = _filled(spec, pages, K, V, page, order)
    for lens, starts in [([90], [N - 90]), ([40, 1, 70], [N - 40, 1500, start - 30])]:
        step = Batch(lens, starts)
        q = torch.randn(sum(lens), H, d, generator=g) * 0.3
        q[:, 0] = direction * 8.0
        q = q.to(dt)
        tables = []
        for n, s in zip(lens, starts):
            table = list(order[: -(-(s + n) // page)])
            for index in range(spec.dead_below(s) // page):
                table[index] = -1
            tables.append(table)
        got = ops.paged_attention(q.to(CUDA), _view(spec, pages, tables, page), step, 0.5, chunk=run, softcap=softcap)
        want = _attention_reference(q.to(F64), K, V, step.positions.cpu(), None, run, 0.5, softcap)
        assert rel(got, want) < 2e-2, (lens, starts)
        if not softcap:
            assert float(got[lens[0] - 1].float().view(H, d)[0].mean()) > 25.0
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv,parts", [(3, 16, 24, None), (2, 64, 32, 2), (5, 12, 20, 1), (3, 5, 7, None),
                                           (4, 128, 128, 4), (1, 32, 16, 1)])
def test_decayed_state_over_portions_and_slots(dtype, H, dk, dv, parts):
    """Two requests in portions of 1 to 37 tokens from state slots that others used before (the engine
    clears a fresh request's slot; here the test does): the state carried in float32 gives the plain
    recurrence over the whole sequence, the columns of a head cut into runs or not."""
    g = torch.Generator().manual_seed(dk * 3 + dv)
    dt = DTYPES[dtype]
    Ta, Tb = 75, 41
    width = 2 * H * dk + 2 * H * dv
    decay = [0.5, 0.9, 0.97, 0.999, 1.0][:H]
    rows = {r: (torch.randn(T, width + 4, generator=g) * 1.5).to(dt) for r, T in (("a", Ta), ("b", Tb))}
    w = 1.0 + 0.2 * torch.randn(H * dv, generator=g)
    S = torch.full((5, H, dk, dv), 3.0, dtype=torch.float32, device=CUDA)
    S[[3, 1]] = 0.0
    got = {"a": [], "b": []}
    cuts = {"a": [0, 37, 38, 40, 56, 75], "b": [0, 1, 18, 19, 20, 41]}
    for i in range(5):
        a0, a1, b0, b1 = cuts["a"][i], cuts["a"][i + 1], cuts["b"][i], cuts["b"][i + 1]
        step = Batch([a1 - a0, b1 - b0], [a0, b0], [3, 1])
        proj = torch.cat([rows["a"][a0:a1], rows["b"][b0:b1]]).to(CUDA)
        out = ops.lightning_attention(proj, 2, 2 + H * dk, 2 + 2 * H * dk, 2 + 2 * H * dk + H * dv, H, dk, dv,
                                      torch.tensor(decay, device=CUDA), w.to(CUDA), 1e-5, S, step, parts=parts)
        got["a"].append(out[: a1 - a0])
        got["b"].append(out[a1 - a0:])
    silu = torch.nn.functional.silu
    for r, T in (("a", Ta), ("b", Tb)):
        x = rows[r].to(F64)[:, 2:]
        q, k = (silu(x[:, i * H * dk: (i + 1) * H * dk]).to(dt).to(F64).view(T, H, dk) for i in (0, 1))
        v = silu(x[:, 2 * H * dk: 2 * H * dk + H * dv]).to(dt).to(F64).view(T, H, dv)
        o, last = plain.decayed_state_heads(q, k, v, decay)
        want = plain.rms(o.reshape(T, H * dv), 1e-5, w.to(F64)) * torch.sigmoid(x[:, 2 * H * dk + H * dv: width])
        assert rel(torch.cat(got[r]), want) < (2e-5 if dtype == "float32" else 1.5e-2), r
        # (in bfloat16 an activation on a rounding boundary may fall the other way than in float64)
        assert rel(S[3 if r == "a" else 1], last) < (2e-5 if dtype == "float32" else 4e-3)
    assert float((S[[0, 2, 4]] - 3.0).abs().max()) == 0.0  # nobody else's slot was touched
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [3, 40, 400])
def test_relu_gated_unit(dtype, rows):
    g = torch.Generator().manual_seed(rows)
    dt = DTYPES[dtype]
    h, gate_up = torch.randn(rows, 128, generator=g).to(dt), (torch.randn(512, 128, generator=g) * 0.2).to(dt)
    got = ops.linear_relu_glu(h.to(CUDA), gate_up.to(CUDA))
    z = h.to(F64) @ gate_up.to(F64).T
    if dtype == "bfloat16":
        z = z.to(dt).to(F64)
    assert rel(got, torch.relu(z[:, :256]) * z[:, 256:]) < (1e-5 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype,tensor_cores", [("float32", False), ("bfloat16", True), ("bfloat16", False)])
@pytest.mark.parametrize("rows,hidden,inner,experts,top,limit", [(50, 96, 24, 5, 2, 0.9), (1, 64, 40, 3, 1, 2.0),
                                                                 (300, 128, 64, 6, 3, 0.5), (1100, 64, 32, 4, 1, 1.0),
                                                                 (7, 100, 20, 3, 3, 0.8)])
def test_table_routed_clamped_experts(dtype, tensor_cores, rows, hidden, inner, experts, top, limit):
    """Experts chosen by a table from token id, each weighing 1 / top, on all three grouped products
    (float32 tiles, mma.sync, and from 1,024 pairs on the tcgen05 kernel's grouped form)."""
    if tensor_cores and (hidden % 8 or inner % 8):
        pytest.skip("the tensor-core products take widths in steps of 8")
    g = torch.Generator().manual_seed(rows + experts)
    dt, vocab = DTYPES[dtype], 37
    h = torch.randn(rows, hidden, generator=g).to(dt)
    W = {"table": torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(vocab)]).to(torch.int32)}
    for e in range(experts):
        W[f"e{e}.gate"], W[f"e{e}.up"] = ((torch.randn(inner, hidden, generator=g) * 0.3).to(dt) for _ in range(2))
        W[f"e{e}.down"] = (torch.randn(hidden, inner, generator=g) * 0.2).to(dt)
    ids = torch.randint(0, vocab, (rows,), generator=g).tolist()
    gate_up = torch.stack([torch.cat([W[f"e{e}.gate"], W[f"e{e}.up"]]) for e in range(experts)]).to(CUDA)
    down = torch.stack([W[f"e{e}.down"] for e in range(experts)]).to(CUDA)
    got = ops.moe_experts(h.to(CUDA), None, None, gate_up, down, top, None, tensor_cores=tensor_cores,
                          table=W["table"].to(CUDA), token_ids=torch.tensor(ids, dtype=torch.int32, device=CUDA),
                          alpha=1.702, limit=limit)
    want = plain.table_experts(h.to(F64), ids, W, "", {"router": {"top": top}, "expert": {"limit": limit}})
    assert rel(got, want) < (2e-5 if dtype == "float32" else 2.5e-2)
    ops.raise_on_error(CUDA)


# ---- the engine -----------------------------------------------------------------------------


def engine_for(name, dtype="float32", page=4, tokens=1024, requests=4, graphs=True, seed=0, raw=None):
    raw = raw or bc.config(name)
    weights = bc.tensors(raw, seed)
    engine = Engine.from_tensors(raw, weights, EngineArgs(dtype=dtype, page_size=page, cache_tokens=tokens,
                                                          max_requests=requests, cuda_graphs=graphs))
    return raw, weights, engine


TOLERANCE = {"float32": 3e-4, "bfloat16": 6e-2}


def assert_rows(got, want, dtype, what="", tolerance=None):
    """Rows of logits against rows of the plain implementation: every row within the tolerance (of the
    largest logit), and in bfloat16 the median row within a quarter of it."""
    tolerance = tolerance or TOLERANCE[dtype]
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    assert got.shape == want.shape
    err = (got - want).abs().amax(-1) / want.abs().max().clamp_min(1e-30)
    assert not torch.isnan(err).any(), what
    assert float(err.max()) < tolerance, (what, int(err.argmax()), float(err.max()))
    if dtype == "bfloat16":
        assert float(err.median()) < tolerance / 4, (what, float(err.median()))


@pytest.mark.parametrize("name", sorted(bc.CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(name, dtype):
    raw, weights, engine = engine_for(name, dtype)
    for n in (1, 2, 3, 41, 230):
        ids = bc.prompt(n, raw["vocab"], n)
        request = engine.cache.open("r")
        got = engine.runner.run([StepEntry(request, ids, list(range(n)))])
        engine.cache.close("r")
        assert_rows(got, plain.forward(ids, weights, raw), dtype, n)
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("name,page", [("K", 4), ("L", 16), ("M", 8), ("N", 16)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_decoding_and_mixed_batches(tmp_path, name, page, dtype):
    """Six requests over four state slots: prompts read whole, in portions of 2 to 9 tokens and
    token by token, decoded tokens beside portions of other requests, requests that end and whose
    pages and slots the next ones take (free pages are filled with NaN before every step)."""
    raw, weights, engine = engine_for(name, dtype, page=page, tokens=448)
    V = raw["vocab"]
    ids = {r: bc.prompt(n, V, i) for i, (r, n) in enumerate({"a": 170, "b": 33, "c": 2, "d": 58, "e": 60, "f": 17}.items())}
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
        assert_rows(logits, plain.forward(ids[r], weights, raw), dtype, r)


@pytest.mark.parametrize("name", ["K", "L", "N"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_decoding_token_by_token(name, dtype):
    """The same prompt whole, and one token a step (captured decode steps, and launched one by one)."""
    for graphs in (True, False):
        raw, weights, engine = engine_for(name, dtype, graphs=graphs)
        ids = bc.prompt(75, raw["vocab"], 77)
        request = engine.cache.open("w")
        whole = engine.runner.run([StepEntry(request, ids, list(range(len(ids))))])
        engine.cache.close("w")
        request = engine.cache.open("t")
        single = torch.cat([engine.runner.run([StepEntry(request, [t], [0])]) for t in ids])
        engine.cache.close("t")
        assert_rows(single, whole, dtype, "token by token against whole", 2e-5 if dtype == "float32" else 4e-2)
        assert_rows(single, plain.forward(ids, weights, raw), dtype)
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_across_tiles_chunks_and_pages(dtype):
    """700 tokens with windows of 150 and 70, runs of 130 and a decay of 0.9999: portions that start and
    end inside tiles of 64 keys, decode chunks of 128 and pages of 16, then 40 tokens decoded beside
    a short request whose pages are the ones the long request gave back."""
    raw, weights, engine = engine_for("M", dtype, page=16, tokens=1024)
    ids = bc.prompt(700, raw["vocab"], 5)
    ids[-1] = ids[11]
    other = bc.prompt(50, raw["vocab"], 6)
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
                torch.stack([expect_b[key[1]] if isinstance(key, tuple) else expect[key] for key in keys]), dtype, keys)
    ops.raise_on_error(CUDA)


def test_the_edges_and_the_constants_show_in_the_logits():
    """One position more or less in a window or a run, a decay, the residual's multiplier or the cap
    moved a little: each moves the plain implementation's logits by far more than the engine is from
    it, so the comparisons above see such a fault. In a prompt and in decoding."""
    raw, weights, engine = engine_for("K", "float32")
    ids = bc.prompt(48, raw["vocab"], 8)
    request = engine.cache.open("r")
    got = [engine.runner.run([StepEntry(request, ids[:30], list(range(30)))])]
    got += [engine.runner.run([StepEntry(request, [t], [0])]) for t in ids[30:]]
    expect = plain.forward(ids, weights, raw)
    assert rel(torch.cat(got), expect) < TOLERANCE["float32"]

    def moved(change):
        other = bc.config("K")
        change(other)
        out = plain.forward(ids, weights, other)
        return min(rel(out[:30], expect[:30]), rel(out[30:], expect[30:]))

    for layer, change in [(1, 1), (1, -1), (2, 1), (2, -1), (3, 1), (3, -1)]:
        assert moved(lambda c: c["layers"][layer]["mixer"]["mask"].update(
            size=c["layers"][layer]["mixer"]["mask"]["size"] + change)) > 1e-3, (layer, change)
    assert moved(lambda c: c["layers"][0]["mixer"]["decay"].__setitem__(2, 0.9)) > 1e-3
    assert moved(lambda c: c.update(residual_mult=0.45)) > 1e-3
    assert moved(lambda c: c["layers"][2]["mixer"].update(softcap=4.0)) > 1e-3
    assert moved(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6)) > 1e-3
    assert moved(lambda c: c["layers"][1]["mlp"]["expert"].update(limit=0.7)) > 1e-3


def test_greedy_generation_long_decoding_and_the_scheduler(tmp_path):
    """Through `load(...).generate`: the scheduler admits, batches and chunks; greedy ids are the plain
    implementation's best, 200 tokens past a two-token prompt included (windows and runs pass over
    decoded tokens many times, the state is carried through all of them)."""
    raw = bc.config("K")
    weights = bc.tensors(raw, 3)
    folder = tmp_path / "m"
    bc.write_folder(folder, raw, weights)
    model = load(folder, dtype="float32", page_size=8, cache_tokens=1024, max_requests=4, max_tokens_per_step=16)
    prompts = [bc.prompt(n, raw["vocab"], 20 + n) for n in (2, 5, 23, 40, 9, 31)]
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

    raw = bc.config("L")
    folder = write_random_model(tmp_path / "m", raw, seed=4)
    weights = {k: (v.float() if v.is_floating_point() else v) for k, v in load_file(str(folder / "model.safetensors")).items()}
    ids = bc.prompt(90, raw["vocab"], 1)
    trace = Trace()
    trace.step({"p": ids[:50]}, want="last")
    trace.step({"p": ids[50:52], "q": ids[:7]})
    for t in range(52, 90):
        trace.step({"p": ids[t: t + 1]}, end=["p"] if t == 89 else ["q"] if t == 52 else [])
    got = trace.run(folder, "bfloat16", tmp_path / "out", vocab=raw["vocab"])
    expect = plain.forward(ids, weights, raw)
    positions, logits = stacked(got["p"])
    assert positions == [49] + list(range(50, 90))
    assert_rows(logits, expect[positions], "bfloat16")
