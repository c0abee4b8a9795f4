"""Narezen as configuration, parts and tensor names.

A decoder whose layers carry, in any order the configuration lists, one of three mixers. Two of them
are pairs of mixers that read the same input and whose outputs are added with a constant each:
`parallel` is a softmax attention without positions whose values are its projected keys, with
weightless per-head RMS norms of queries and keys and a learned sink per head, beside a linear
attention whose state decays by a factor per key channel that the token sets through a low-rank map
(alpha = sigmoid(z)^(1/tau)); `parallel_2` is a softmax attention with rotated queries and keys and
a one in the denominator, beside a retention: linear attention with a constant decay per head,
rotated queries and keys, keys times dim^-1/2. The third, `rglru`, is a recurrent block with a
real-gated linear recurrence behind a short convolution. Every branch sits between two RMS norms:
x += after(branch(before(x))). The feed-forward is a mixture of small gated units chosen by sigmoid
scores, the chosen expert being given the token times its score, plus a shared expert; a layer may
have none. The embedding is scaled; the head has its own matrix and the logits are soft-capped.
Everything here is data for the generic engine.

config.json keys: `architecture` ("Narezen"), `vocab`, `width`, `embedding.scale`, `norm.eps`,
`logit_softcap`, and `layers`: a list of {`type`: "parallel" | "parallel_2" | "rglru", `mixer`,
`mlp`: null | {kind: "moe", expert {ff}, router {experts, top}, shared {ff}}} with `mixer` =
{left {heads, kv_heads, dim, vdim, scale, rot? {base, dims}}, right {heads, dim, vdim, tau | decay
[heads], rot? {base, dims}}, left_scale, right_scale} for the pairs and {width, blocks, conv} for rglru.
Tensor names: `embed`, `head`, `final.norm`, and per layer i `l<i>.norm1|norm1b|norm2|norm2b`,
`l<i>.mix.left.q|k|o` (+ `.sink`, or `.v`), `l<i>.mix.right.q|k|v|g|o` (+ `.norm`, `.a1`, `.a2`,
`.a2.b`), or `l<i>.mix.x|x.b|y|y.b|conv|conv.b|ra|ra.b|ri|ri.b|lam|o`; `l<i>.mlp.router`,
`l<i>.mlp.e<j>.gate|up|down`, `l<i>.mlp.shared.gate|up|down`.
"""

from __future__ import annotations

import dataclasses
import re
from dataclasses import dataclass
from typing import Any, Callable

import torch

from mlx_omnia_b200.config.hydrate import ConfigError
from mlx_omnia_b200.parts.base import PartSpec
from mlx_omnia_b200.parts.model import LayerSpec, ModelSpec, ScheduleEntry
from mlx_omnia_b200.registry import Architecture, register_architecture

RECURRENCE_DECAY = 8.0  # c in a = exp(-c r softplus(lam)) of the gated recurrence
DEFAULT_DECAY_RANK = 16  # inner width of a decay map in random weights made without a checkpoint to read it from

PAIR, PAIR_2, RECURRENT = "parallel", "parallel_2", "rglru"


@dataclass(frozen=True)
class NarezenAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int = 0
    rot_base: float = 0.0


@dataclass(frozen=True)
class NarezenState:
    heads: int
    dim: int
    vdim: int
    tau: float | None = None  # a decay per key channel through a low-rank map ...
    decay_rank: int = 0  # ... whose inner width only the tensors give
    decay: tuple[float, ...] | None = None  # or a constant per head
    rot_dims: int = 0
    rot_base: float = 0.0


@dataclass(frozen=True)
class NarezenMixer:
    type: str
    left: NarezenAttention | None = None
    right: NarezenState | None = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    width: int = 0  # rglru
    blocks: int = 0
    conv: int = 0


@dataclass(frozen=True)
class NarezenFeedForward:
    ff: int
    experts: int
    top: int
    shared_ff: int | None


@dataclass(frozen=True)
class NarezenConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: float | None
    mixers: tuple[NarezenMixer, ...]
    feed_forwards: tuple[NarezenFeedForward | None, ...]


def _need(raw: Any, key: str, where: str):
    if not isinstance(raw, dict) or key not in raw:
        raise ConfigError(f"Narezen: {where} lacks the key {key!r}")
    return raw[key]


def _rot(raw: dict, dim: int, where: str) -> tuple[int, float]:
    rot = raw.get("rot")
    if rot is None:
        return 0, 0.0
    dims = int(_need(rot, "dims", where + ".rot"))
    if dims % 2 or not 0 <= dims <= dim:
        raise ConfigError(f"Narezen: {where}.rot.dims must be even and at most dim = {dim}, got {dims}")
    return dims, (float(_need(rot, "base", where + ".rot")) if dims else 0.0)


def _attention(raw: dict, where: str, rotated: bool) -> NarezenAttention:
    heads, kv_heads, dim, vdim = (int(_need(raw, key, where)) for key in ("heads", "kv_heads", "dim", "vdim"))
    if kv_heads < 1 or heads % kv_heads:
        raise ConfigError(f"Narezen: {where}: {heads} heads do not divide into {kv_heads} key/value heads")
    if not rotated and vdim != dim:
        raise ConfigError(f"Narezen: {where}: values that are the keys have the keys' size {dim}, not {vdim}")
    dims, base = _rot(raw, dim, where) if rotated else (0, 0.0)
    return NarezenAttention(heads, kv_heads, dim, vdim, float(_need(raw, "scale", where)), dims, base)


def _state(raw: dict, where: str, kind: str) -> NarezenState:
    heads, dim, vdim = (int(_need(raw, key, where)) for key in ("heads", "dim", "vdim"))
    if kind == PAIR:
        tau = float(_need(raw, "tau", where))
        if tau <= 0:
            raise ConfigError(f"Narezen: {where}.tau must be positive, got {tau}")
        return NarezenState(heads, dim, vdim, tau=tau)
    decay = tuple(float(d) for d in _need(raw, "decay", where))
    if len(decay) != heads:
        raise ConfigError(f"Narezen: {where}.decay has {len(decay)} entries for {heads} heads")
    dims, base = _rot(raw, dim, where)
    return NarezenState(heads, dim, vdim, decay=decay, rot_dims=dims, rot_base=base)


def _mixer(kind: str, raw: dict, where: str) -> NarezenMixer:
    if kind == RECURRENT:
        width, blocks, conv = (int(_need(raw, key, where)) for key in ("width", "blocks", "conv"))
        if blocks < 1 or width % blocks:
            raise ConfigError(f"Narezen: {where}: {width} channels do not divide into {blocks} blocks")
        if conv < 1:
            raise ConfigError(f"Narezen: {where}.conv must be at least 1, got {conv}")
        return NarezenMixer(kind, width=width, blocks=blocks, conv=conv)
    return NarezenMixer(kind, _attention(_need(raw, "left", where), where + ".left", kind == PAIR_2),
                        _state(_need(raw, "right", where), where + ".right", kind),
                        float(raw.get("left_scale", 1.0)), float(raw.get("right_scale", 1.0)))


def _feed_forward(raw: dict | None, where: str) -> NarezenFeedForward | None:
    if raw is None:
        return None
    kind = _need(raw, "kind", where)
    if kind != "moe":
        raise ConfigError(f"Narezen: {where} has the unknown kind {kind!r}")
    router, shared = _need(raw, "router", where), raw.get("shared")
    experts, top = int(_need(router, "experts", where + ".router")), int(_need(router, "top", where + ".router"))
    if experts < 1 or not 1 <= top <= experts:
        raise ConfigError(f"Narezen: {where}.router: {top} of {experts} experts")
    return NarezenFeedForward(int(_need(_need(raw, "expert", where), "ff", where + ".expert")), experts, top,
                              None if shared is None else int(_need(shared, "ff", where + ".shared")))


def parse(raw: dict[str, Any]) -> NarezenConfig:
    if raw.get("architecture") != "Narezen":
        raise ConfigError(f"expected architecture 'Narezen', got {raw.get('architecture')!r}")
    mixers, feed_forwards = [], []
    for index, layer in enumerate(_need(raw, "layers", "config.json")):
        where = f"layers[{index}]"
        kind = _need(layer, "type", where)
        if kind not in (PAIR, PAIR_2, RECURRENT):
            raise ConfigError(f"Narezen: {where} has the unknown type {kind!r}")
        mixers.append(_mixer(kind, _need(layer, "mixer", where), where + ".mixer"))
        feed_forwards.append(_feed_forward(layer.get("mlp"), where + ".mlp"))
    if not mixers:
        raise ConfigError("Narezen: no layers")
    cap = raw.get("logit_softcap")
    return NarezenConfig(vocab=int(_need(raw, "vocab", "config.json")), width=int(_need(raw, "width", "config.json")),
                         norm_eps=float(_need(_need(raw, "norm", "config.json"), "eps", "norm")),
                         embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                         logit_softcap=None if cap is None else float(cap),
                         mixers=tuple(mixers), feed_forwards=tuple(feed_forwards))


def sizes_from_tensors(config: NarezenConfig, shape_of: Callable[[str], tuple[int, ...] | None]) -> NarezenConfig:
    """The inner width of a decay's low-rank map is the rows of its first matrix; no key names it."""
    mixers = []
    for index, m in enumerate(config.mixers):
        if m.right is not None and m.right.decay is None:
            shape = shape_of(f"l{index}.mix.right.a1")
            if shape is not None:
                m = dataclasses.replace(m, right=dataclasses.replace(m.right, decay_rank=int(shape[0])))
        mixers.append(m)
    return dataclasses.replace(config, mixers=tuple(mixers))


def _norm(config: NarezenConfig) -> PartSpec:
    return PartSpec("rms_norm", {"size": config.width, "eps": config.norm_eps, "weight": "plain"})


def _mixer_spec(config: NarezenConfig, m: NarezenMixer) -> PartSpec:
    if m.type == RECURRENT:
        return PartSpec("gated_channel_recurrence", {"hidden": config.width, "width": m.width, "blocks": m.blocks,
                                                     "conv": m.conv, "c_decay": RECURRENCE_DECAY})
    a, s = m.left, m.right
    attention = {"hidden": config.width, "heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim,
                 "scale": a.scale}
    state = {"hidden": config.width, "heads": s.heads, "dim": s.dim, "vdim": s.vdim, "norm_eps": config.norm_eps}
    if m.type == PAIR:
        attention.update({"norm_eps": config.norm_eps, "norm_weight": False, "sink": True, "values": "keys"})
        state.update({"decay": None, "decay_rank": max(s.decay_rank, 1), "tau": s.tau, "q_scale": s.dim ** -0.5,
                      "norm_weight": True})
    else:
        rotary = lambda dims, base: PartSpec("rotary", {"dims": dims, "theta": base}) if dims else None  # noqa: E731
        attention.update({"sink": "zero", "position": rotary(a.rot_dims, a.rot_base)})
        state.update({"decay": s.decay, "position": rotary(s.rot_dims, s.rot_base), "k_scale": s.dim ** -0.5,
                      "norm_weight": False})
    return PartSpec("side_by_side", {"left": PartSpec("sink_window_attention", attention),
                                     "right": PartSpec("gated_state_attention", state),
                                     "left_scale": m.left_scale, "right_scale": m.right_scale})


def model_spec(config: NarezenConfig) -> ModelSpec:
    layers = []
    for index, (m, f) in enumerate(zip(config.mixers, config.feed_forwards)):
        feed_forward = None
        if f is not None:
            feed_forward = PartSpec("routed_experts", {"hidden": config.width, "inner": f.ff, "experts": f.experts,
                                                       "top": f.top, "correction": False, "scoring": "sigmoid",
                                                       "weigh": "input", "shared_inner": f.shared_ff})
        names = ("norm1", "norm1b") if feed_forward is None else ("norm1", "norm1b", "norm2", "norm2b")
        block = PartSpec("scaled_sandwich", {"mixer": _mixer_spec(config, m), "feed_forward": feed_forward,
                                             "norms": {name: _norm(config) for name in names}})
        layers.append(LayerSpec(block, f"l{index}"))
    return ModelSpec(
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "hidden": config.width,
                                               "scale": config.embedding_scale}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=_norm(config),
        head=PartSpec("lm_head", {"vocab": config.vocab, "hidden": config.width, "softcap": config.logit_softcap}),
        embedding_prefix="embed", final_norm_prefix="final.norm", head_prefix="head",
    )


_WEIGHT_SUFFIXED = re.compile(r"^(embed|head|final\.norm|l\d+\.norm(1|1b|2|2b))$")


def tensor_name(file_name: str) -> str:
    """The file's names are the model's, but for the parts that call their one tensor `weight`."""
    return file_name + ".weight" if _WEIGHT_SUFFIXED.match(file_name) else file_name


def random_tensors(config: NarezenConfig, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors under the checkpoint's names, drawn on the CPU in a fixed order from one
    generator: matrices N(0, gain / sqrt(fan_in)); norm weights around one; sinks, biases and the
    recurrence's parameters of a size that makes every mechanism count."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape: int, std: float = 1.0) -> torch.Tensor:
        return torch.randn(*shape, generator=g, dtype=torch.float32) * std

    def matrix(rows: int, cols: int, gain: float = 1.0) -> torch.Tensor:
        return normal(rows, cols, std=gain * cols ** -0.5)

    D = config.width
    out = {"embed": normal(config.vocab, D), "head": matrix(config.vocab, D)}
    for i, (m, f) in enumerate(zip(config.mixers, config.feed_forwards)):
        p = f"l{i}."
        out[p + "norm1"], out[p + "norm1b"] = 1.0 + normal(D, std=0.1), 1.0 + normal(D, std=0.1)
        if m.type == RECURRENT:
            w, bw = m.width, m.width // m.blocks
            q = p + "mix."
            out[q + "x"], out[q + "y"] = matrix(w, D, gain=2.0), matrix(w, D, gain=2.0)
            out[q + "x.b"], out[q + "y.b"] = normal(w, std=0.2), normal(w, std=0.2)
            out[q + "conv"], out[q + "conv.b"] = normal(w, m.conv, std=m.conv ** -0.5), normal(w, std=0.1)
            out[q + "ra"], out[q + "ri"] = normal(m.blocks, bw, bw, std=bw ** -0.5), normal(m.blocks, bw, bw, std=bw ** -0.5)
            out[q + "ra.b"], out[q + "ri.b"] = normal(m.blocks, bw, std=0.5), normal(m.blocks, bw, std=0.5)
            out[q + "lam"] = normal(w, std=1.0) - 2.0
            out[q + "o"] = matrix(D, w)
        else:
            a, s = m.left, m.right
            q = p + "mix.left."
            out[q + "q"], out[q + "k"] = matrix(a.heads * a.dim, D, gain=2.0), matrix(a.kv_heads * a.dim, D, gain=2.0)
            if m.type == PAIR:
                out[q + "sink"] = normal(a.heads)
            else:
                out[q + "v"] = matrix(a.kv_heads * a.vdim, D, gain=2.0)
            out[q + "o"] = matrix(D, a.heads * a.vdim)
            q = p + "mix.right."
            out[q + "q"], out[q + "k"] = matrix(s.heads * s.dim, D, gain=2.0), matrix(s.heads * s.dim, D, gain=2.0)
            out[q + "v"], out[q + "g"] = matrix(s.heads * s.vdim, D, gain=2.0), matrix(s.heads * s.vdim, D)
            out[q + "o"] = matrix(D, s.heads * s.vdim)
            if m.type == PAIR:
                rank = s.decay_rank or DEFAULT_DECAY_RANK
                out[q + "norm"] = 1.0 + normal(s.vdim, std=0.1)
                out[q + "a1"], out[q + "a2"] = matrix(rank, D), matrix(s.heads * s.dim, rank, gain=2.0)
                out[q + "a2.b"] = normal(s.heads * s.dim, std=0.5) + 2.0
        if f is None:
            continue
        out[p + "norm2"], out[p + "norm2b"] = 1.0 + normal(D, std=0.1), 1.0 + normal(D, std=0.1)
        out[p + "mlp.router"] = matrix(f.experts, D, gain=2.0)
        names = [f"e{e}" for e in range(f.experts)] + (["shared"] if f.shared_ff is not None else [])
        for name in names:
            inner = f.shared_ff if name == "shared" else f.ff
            out[p + f"mlp.{name}.gate"], out[p + f"mlp.{name}.up"] = matrix(inner, D, gain=2.0), matrix(inner, D, gain=2.0)
            out[p + f"mlp.{name}.down"] = matrix(D, inner)
    out["final.norm"] = 1.0 + normal(D, std=0.1)
    return out


ARCHITECTURE = Architecture(
    name="narezen",
    config_class=NarezenConfig,
    parse=parse,
    model_spec=model_spec,
    tensor_name=tensor_name,
    random_tensors=random_tensors,
    sizes_from_tensors=sizes_from_tensors,
)

register_architecture(ARCHITECTURE, "Narezen", "narezen")
