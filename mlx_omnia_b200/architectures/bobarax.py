"""Bobarax as configuration, parts and tensor names.

A decoder whose layers, in any order the configuration lists, carry one of three mixers: linear
attention with a constant decay per head and a state carried from token to token (`lightning`); a
softmax attention without positions whose queries look back to the start of their own run of
positions, with scores capped by a tanh (`attention`); and a sliding-window softmax attention with an
interleaved rotation of part of every head and a sigmoid gate on the heads' outputs (`attention_2`),
which may carry no key/value tensors and read an earlier layer's cache instead (`kv_from`). Queries
and keys of both attentions are RMS-normed over the whole projection at once. Every branch sits
between two norms with weights stored around zero, and enters the residual multiplied by a constant:
x += m * after(branch(before(x))). The feed-forward is a relu-gated unit, or a mixture of small
clamped gated units that a table from token id to experts chooses among (no router); a layer may have
none. The head reads the embedding table; the logits are scaled. Everything here is data for the
generic engine.

config.json keys: `architecture` ("Bobarax"), `vocab`, `width`, `residual_mult`, `logit_scale`,
`norm.eps`, and `layers`: a list of {`type`: "lightning" | "attention" | "attention_2", `mixer`,
`mlp`: null | {kind: "dense", ff} | {kind: "moe", expert {ff, limit}, router {experts, top}}} with
`mixer` = {heads, dim, vdim, decay [heads]} for lightning, {heads, kv_heads, dim, vdim, scale,
softcap?, mask {size}} for attention, {heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask
{size}, kv_from?} for attention_2.
Tensor names: `embed`, `final.norm`, and per layer i `l<i>.norm1|norm1b|norm2|norm2b`,
`l<i>.mix.q|k|v|o` (+ `.q.norm`, `.k.norm` for the attentions, `.g` for attention_2 and lightning,
`.norm` for lightning), `l<i>.mlp.gate|up|down` or `l<i>.mlp.table`, `l<i>.mlp.e<j>.gate|up|down`.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any

import torch

from mlx_omnia_b200.config.hydrate import ConfigError
from mlx_omnia_b200.parts.base import PartSpec
from mlx_omnia_b200.parts.model import LayerSpec, ModelSpec, ScheduleEntry
from mlx_omnia_b200.registry import Architecture, register_architecture

EXPERT_SLOPE = 1.702  # of the sigmoid in an expert's gated unit

LIGHTNING, CHUNKED, WINDOWED = "lightning", "attention", "attention_2"


@dataclass(frozen=True)
class BobaraxMixer:
    type: str
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0  # the attentions
    scale: float = 1.0
    mask: int | None = None  # run length (attention) or window (attention_2); None: every earlier position
    softcap: float | None = None  # attention
    rot_dims: int = 0  # attention_2
    rot_base: float = 0.0
    kv_from: int | None = None
    decay: tuple[float, ...] = ()  # lightning


@dataclass(frozen=True)
class BobaraxFeedForward:
    kind: str  # "dense" or "moe"
    ff: int
    limit: float = 0.0  # moe
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class BobaraxConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_scale: float
    mixers: tuple[BobaraxMixer, ...]
    feed_forwards: tuple[BobaraxFeedForward | None, ...]


def _need(raw: Any, key: str, where: str):
    if not isinstance(raw, dict) or key not in raw:
        raise ConfigError(f"Bobarax: {where} lacks the key {key!r}")
    return raw[key]


def _mixer(kind: str, raw: dict, where: str, index: int) -> BobaraxMixer:
    heads, dim, vdim = (int(_need(raw, key, where)) for key in ("heads", "dim", "vdim"))
    if kind == LIGHTNING:
        decay = tuple(float(d) for d in _need(raw, "decay", where))
        if len(decay) != heads:
            raise ConfigError(f"Bobarax: {where}.decay has {len(decay)} entries for {heads} heads")
        return BobaraxMixer(kind, heads, dim, vdim, decay=decay)
    kv_heads = int(_need(raw, "kv_heads", where))
    if kv_heads < 1 or heads % kv_heads:
        raise ConfigError(f"Bobarax: {where}: {heads} heads do not divide into {kv_heads} key/value heads")
    mask = raw.get("mask")
    size = None if mask is None else int(_need(mask, "size", where + ".mask"))
    if size is not None and size < 1:
        raise ConfigError(f"Bobarax: {where}.mask.size must be at least 1, got {size}")
    scale = float(_need(raw, "scale", where))
    if kind == CHUNKED:
        softcap = raw.get("softcap")
        return BobaraxMixer(kind, heads, dim, vdim, kv_heads, scale, size, None if softcap is None else float(softcap))
    rot = raw.get("rot")
    dims = 0 if rot is None else int(_need(rot, "dims", where + ".rot"))
    if dims % 2 or not 0 <= dims <= dim:
        raise ConfigError(f"Bobarax: {where}.rot.dims must be even and at most dim = {dim}, got {dims}")
    kv_from = raw.get("kv_from")
    if kv_from is not None and not 0 <= int(kv_from) < index:
        raise ConfigError(f"Bobarax: {where}.kv_from names layer {kv_from}, which does not run before layer {index}")
    return BobaraxMixer(kind, heads, dim, vdim, kv_heads, scale, size, rot_dims=dims,
                        rot_base=float(_need(rot, "base", where + ".rot")) if dims else 0.0,
                        kv_from=None if kv_from is None else int(kv_from))


def _feed_forward(raw: dict | None, where: str) -> BobaraxFeedForward | None:
    if raw is None:
        return None
    kind = _need(raw, "kind", where)
    if kind == "dense":
        return BobaraxFeedForward("dense", int(_need(raw, "ff", where)))
    if kind == "moe":
        expert, router = _need(raw, "expert", where), _need(raw, "router", where)
        return BobaraxFeedForward("moe", int(_need(expert, "ff", where + ".expert")),
                                  limit=float(_need(expert, "limit", where + ".expert")),
                                  experts=int(_need(router, "experts", where + ".router")),
                                  top=int(_need(router, "top", where + ".router")))
    raise ConfigError(f"Bobarax: {where} has the unknown kind {kind!r}")


def parse(raw: dict[str, Any]) -> BobaraxConfig:
    if raw.get("architecture") != "Bobarax":
        raise ConfigError(f"expected architecture 'Bobarax', got {raw.get('architecture')!r}")
    mixers, feed_forwards = [], []
    for index, layer in enumerate(_need(raw, "layers", "config.json")):
        where = f"layers[{index}]"
        kind = _need(layer, "type", where)
        if kind not in (LIGHTNING, CHUNKED, WINDOWED):
            raise ConfigError(f"Bobarax: {where} has the unknown type {kind!r}")
        mixers.append(_mixer(kind, _need(layer, "mixer", where), where + ".mixer", index))
        feed_forwards.append(_feed_forward(layer.get("mlp"), where + ".mlp"))
    if not mixers:
        raise ConfigError("Bobarax: no layers")
    for index, mixer in enumerate(mixers):
        if mixer.kv_from is None:
            continue
        owner = mixers[mixer.kv_from]
        if owner.type != WINDOWED or owner.kv_from is not None:
            raise ConfigError(f"Bobarax: layers[{index}] reads the cache of layer {mixer.kv_from}, which has none of its kind")
        if (owner.kv_heads, owner.dim, owner.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
            raise ConfigError(f"Bobarax: layers[{index}] and the layer whose cache it reads differ in key/value sizes")
    return BobaraxConfig(vocab=int(_need(raw, "vocab", "config.json")), width=int(_need(raw, "width", "config.json")),
                         norm_eps=float(_need(_need(raw, "norm", "config.json"), "eps", "norm")),
                         residual_mult=float(raw.get("residual_mult", 1.0)), logit_scale=float(raw.get("logit_scale", 1.0)),
                         mixers=tuple(mixers), feed_forwards=tuple(feed_forwards))


def _norm(config: BobaraxConfig) -> PartSpec:
    return PartSpec("rms_norm", {"size": config.width, "eps": config.norm_eps, "weight": "centred"})


def _mixer_spec(config: BobaraxConfig, m: BobaraxMixer) -> PartSpec:
    if m.type == LIGHTNING:
        return PartSpec("decay_attention", {"hidden": config.width, "heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                            "decay": m.decay, "norm_eps": config.norm_eps})
    common = {"hidden": config.width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
              "scale": m.scale, "norm_eps": config.norm_eps, "norm_over": "projection"}
    if m.type == CHUNKED:
        return PartSpec("sink_window_attention", {**common, "chunk": m.mask, "softcap": m.softcap})
    position = PartSpec("rotary", {"dims": m.rot_dims, "theta": m.rot_base, "pairing": "interleaved"}) if m.rot_dims else None
    return PartSpec("sink_window_attention", {**common, "window": m.mask, "position": position, "gated": True,
                                              "own_kv": m.kv_from is None})


def model_spec(config: BobaraxConfig) -> ModelSpec:
    layers = []
    for index, (m, f) in enumerate(zip(config.mixers, config.feed_forwards)):
        if f is None:
            feed_forward = None
        elif f.kind == "dense":
            feed_forward = PartSpec("relu_glu_mlp", {"hidden": config.width, "inner": f.ff})
        else:
            feed_forward = PartSpec("table_experts", {"hidden": config.width, "inner": f.ff, "experts": f.experts,
                                                      "top": f.top, "vocab": config.vocab, "limit": f.limit,
                                                      "alpha": EXPERT_SLOPE})
        names = ("norm1", "norm1b") if feed_forward is None else ("norm1", "norm1b", "norm2", "norm2b")
        block = PartSpec("scaled_sandwich", {"mixer": _mixer_spec(config, m), "feed_forward": feed_forward,
                                             "norms": {name: _norm(config) for name in names},
                                             "branch_scale": config.residual_mult})
        layers.append(LayerSpec(block, f"l{index}"))
    return ModelSpec(
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "hidden": config.width}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, m.kv_from) for i, m in enumerate(config.mixers)),
        final_norm=_norm(config),
        head=PartSpec("lm_head", {"vocab": config.vocab, "hidden": config.width, "tied": True,
                                  "multiplier": config.logit_scale}),
        embedding_prefix="embed", final_norm_prefix="final.norm", head_prefix="head",
    )


_WEIGHT_SUFFIXED = re.compile(r"^(embed|final\.norm|l\d+\.norm(1|1b|2|2b))$")


def tensor_name(file_name: str) -> str:
    """The file's names are the model's, but for the parts that call their one tensor `weight`."""
    return file_name + ".weight" if _WEIGHT_SUFFIXED.match(file_name) else file_name


def random_tensors(config: BobaraxConfig, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors (and int32 tables) under the checkpoint's names, drawn on the CPU in a fixed order
    from one generator: matrices N(0, gain / sqrt(fan_in)); the block norms' weights around zero;
    the attentions' and the output norm's weights around one; every table row `top` different experts."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape: int, std: float = 1.0) -> torch.Tensor:
        return torch.randn(*shape, generator=g, dtype=torch.float32) * std

    def matrix(rows: int, cols: int, gain: float = 1.0) -> torch.Tensor:
        return normal(rows, cols, std=gain * cols ** -0.5)

    D = config.width
    out = {"embed": normal(config.vocab, D)}
    for i, (m, f) in enumerate(zip(config.mixers, config.feed_forwards)):
        p = f"l{i}."
        out[p + "norm1"], out[p + "norm1b"] = normal(D, std=0.1), normal(D, std=0.1)
        H, dk, dv = m.heads, m.dim, m.vdim
        if m.type == LIGHTNING:
            out[p + "mix.q"], out[p + "mix.k"] = matrix(H * dk, D, gain=2.0), matrix(H * dk, D, gain=2.0)
            out[p + "mix.v"], out[p + "mix.g"] = matrix(H * dv, D, gain=2.0), matrix(H * dv, D)
            out[p + "mix.norm"] = 1.0 + normal(H * dv, std=0.1)
        else:
            out[p + "mix.q"] = matrix(H * dk, D, gain=2.0)
            out[p + "mix.q.norm"] = 1.0 + normal(H * dk, std=0.2)
            if m.kv_from is None:
                out[p + "mix.k"], out[p + "mix.v"] = matrix(m.kv_heads * dk, D, gain=2.0), matrix(m.kv_heads * dv, D, gain=2.0)
                out[p + "mix.k.norm"] = 1.0 + normal(m.kv_heads * dk, std=0.2)
            if m.type == WINDOWED:
                out[p + "mix.g"] = matrix(H * dv, D)
        out[p + "mix.o"] = matrix(D, H * dv)
        if f is None:
            continue
        out[p + "norm2"], out[p + "norm2b"] = normal(D, std=0.1), normal(D, std=0.1)
        if f.kind == "dense":
            out[p + "mlp.gate"], out[p + "mlp.up"] = matrix(f.ff, D, gain=2.0), matrix(f.ff, D, gain=2.0)
            out[p + "mlp.down"] = matrix(D, f.ff)
        else:
            for e in range(f.experts):
                out[p + f"mlp.e{e}.gate"], out[p + f"mlp.e{e}.up"] = matrix(f.ff, D, gain=2.0), matrix(f.ff, D, gain=2.0)
                out[p + f"mlp.e{e}.down"] = matrix(D, f.ff)
            rows = [torch.randperm(f.experts, generator=g)[: f.top] for _ in range(config.vocab)]
            out[p + "mlp.table"] = torch.stack(rows).to(torch.int32)
    out["final.norm"] = normal(D, std=0.1)
    return out


ARCHITECTURE = Architecture(
    name="bobarax",
    config_class=BobaraxConfig,
    parse=parse,
    model_spec=model_spec,
    tensor_name=tensor_name,
    random_tensors=random_tensors,
)

register_architecture(ARCHITECTURE, "Bobarax", "bobarax")
