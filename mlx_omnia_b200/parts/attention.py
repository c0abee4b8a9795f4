"""Attention mixers over the paged cache.

Reference: separate q/k/v projections, per-head norm before rotation, keys cached after
rotation, grouped-query softmax attention, a full-width sigmoid gate computed from the
same input as q, output projection (src/mlx_omnia/engine/core/attention.py:618-682);
Muse-Glimmer's choice of options
(src/mlx_omnia/engine/models/muse_glimmer/layers/attention.py:20-47).
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import POSITIONS, KVSpec, Mixer, PartSpec, TensorSpec, register_mixer


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    """Grouped-query causal attention.

    hidden, heads, kv_heads, head_dim: sizes (heads * head_dim need not equal hidden)
    scale:     multiplies q.k before the softmax
    window:    None, or how many latest positions (the query's own included) are visible
    qk_norm_eps: None, or the eps of a weightless RMS norm of every q and k head
    gated:     multiply the attention output by sigmoid(gate_proj(h)), full width
    position:  PartSpec of the position encoding applied to q and k
    own_kv:    False for a layer that only reads another layer's cache (no k/v weights)
    """

    graph_safe = True  # no host-side work per request: a decode step can be captured
    graph_safe_mixed = True  # nor in a step of any other shape: repeated mixed steps can be captured too
    takes_pending = True  # h goes to the in-projection and nowhere else

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, scale: float,
                 window: int | None = None, qk_norm_eps: float | None = None, gated: bool = False,
                 position: PartSpec | None = None, own_kv: bool = True) -> None:
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads do not divide into {kv_heads} groups")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"head_dim must be even and at most 256, got {head_dim}")
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.scale, self.window, self.qk_norm_eps, self.gated, self.own_kv = scale, window, qk_norm_eps, gated, own_kv
        self.position = POSITIONS.build(position or PartSpec("none"))
        if getattr(self.position, "pairing", "half") != "half":
            raise ValueError("gqa_attention rotates half-split pairs")

    def kv_spec(self) -> KVSpec:
        return KVSpec.keys_and_values(self.kv_heads, self.head_dim, self.window)

    def tensors(self) -> dict[str, TensorSpec]:
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        specs = {"q_proj.weight": TensorSpec((q, self.hidden)), "o_proj.weight": TensorSpec((self.hidden, q))}
        if self.gated:
            specs["gate_proj.weight"] = TensorSpec((q, self.hidden))
        if self.own_kv:
            specs["k_proj.weight"] = TensorSpec((kv, self.hidden))
            specs["v_proj.weight"] = TensorSpec((kv, self.hidden))
        return specs

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.position.load({}, runtime)
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        # One operand [q | gate | k | v] so the step runs a single input projection.
        rows, self.q_col, col = [tensors["q_proj.weight"]], 0, q
        self.gate_col = self.k_col = self.v_col = 0
        if self.gated:
            rows.append(tensors["gate_proj.weight"])
            self.gate_col, col = col, col + q
        if self.own_kv:
            rows += [tensors["k_proj.weight"], tensors["v_proj.weight"]]
            self.k_col, self.v_col = col, col + kv
        self.in_proj = torch.cat(rows, dim=0).contiguous()
        self.o_proj = tensors["o_proj.weight"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        if ctx.kv is None:
            raise RuntimeError("an attention mixer needs cache pages")
        if ctx.kv.writes and not self.own_kv:
            raise RuntimeError("a mixer without k/v projections cannot own a cache entry")
        inv_freq = self.position.table()
        # Many rows: the product's epilogue normalises, rotates and stores (only the gate's columns of
        # the projected rows are then written).
        made = ops.linear_qkv(h, self.in_proj, self.q_col, self.k_col, self.v_col, self.heads,
                              self.kv_heads if self.own_kv else 0, self.head_dim, self.qk_norm_eps, inv_freq, ctx.step,
                              ctx.kv if self.own_kv else None)
        if made is not None:
            proj, q = made
            out = ops.paged_attention(q, ctx.kv, ctx.step, self.scale, gate=proj if self.gated else None,
                                      gate_col=self.gate_col)
            return ops.linear(out, self.o_proj)
        proj = ops.linear(h, self.in_proj)
        gate = proj if self.gated else None
        if self.own_kv and ops.decode_fusable(proj, self.heads, self.kv_heads, self.head_dim, inv_freq, ctx.kv,
                                              ctx.step):
            # Single tokens only: the attention kernel normalises, rotates and stores by itself.
            rows = ops.Projection(proj, self.q_col, self.k_col, self.v_col, self.heads, self.head_dim,
                                  self.qk_norm_eps, inv_freq)
            out = ops.paged_attention(None, ctx.kv, ctx.step, self.scale, gate=gate, gate_col=self.gate_col,
                                      projection=rows)
        else:
            q = ops.qk_norm_rope_store(proj, self.q_col, self.k_col, self.v_col, self.heads, self.kv_heads,
                                       self.head_dim, self.qk_norm_eps, inv_freq, ctx.step.positions,
                                       ctx.kv if self.own_kv else None)
            out = ops.paged_attention(q, ctx.kv, ctx.step, self.scale, gate=gate, gate_col=self.gate_col)
        return ops.linear(out, self.o_proj)


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """Causal attention whose keys and values are expanded from one low-rank row per position.

    hidden, heads: sizes; dim: unrotated query/key dims per head; rot_dim: rotated ones (a query head
    is laid out [dim | rot_dim]); vdim: value dims per head; kv_rank: width of the latent.
    The down projection gives kv_rank + rot_dim numbers per token: the first kv_rank, RMS-normed
    (`dkv.norm`, eps `norm_eps`), are the latent c; the last rot_dim, rotated, are one key part that
    all heads share. Head h's key is [uk_h c | shared part], its value uv_h c; only [c | shared part]
    is cached, one row per position. This engine never expands the cache: uk is folded into the query
    (q_lat = uk_h^T q_plain) and uv applied to the attention's output in latent space.
    scale:    multiplies the scores
    position: a rotary part with interleaved pairing over the first `dims` of the rot_dim
    sink:     the softmax's denominator also holds exp(sink_h) (tensor `sink` [heads], unscaled)
    gated:    head h's output is multiplied by sigmoid(g(h))_h (tensor `g` [heads, hidden])
    window:   None, or how many latest positions are visible

    Tensors: q [heads * (dim + rot_dim), hidden]; dkv [kv_rank + rot_dim, hidden]; dkv.norm [kv_rank];
    uk [heads * dim, kv_rank]; uv [heads * vdim, kv_rank]; o [hidden, heads * vdim]."""

    graph_safe = True
    graph_safe_mixed = True

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 norm_eps: float, position: PartSpec, sink: bool = True, gated: bool = True,
                 window: int | None = None) -> None:
        if kv_rank > ops.LATENT_MAX_RANK:
            raise ValueError(f"latent_attention takes a latent of at most {ops.LATENT_MAX_RANK}")
        self.hidden, self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank = hidden, heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.norm_eps, self.sink, self.gated, self.window = float(scale), float(norm_eps), sink, gated, window
        self.position = POSITIONS.build(position)
        if getattr(self.position, "pairing", None) != "interleaved":
            raise ValueError("latent_attention rotates interleaved pairs")
        if self.position.dims > rot_dim:
            raise ValueError(f"{self.position.dims} rotary dims do not fit a rotated part of {rot_dim}")

    def kv_spec(self) -> KVSpec:
        return KVSpec(((1, self.kv_rank + self.rot_dim),), self.window)

    def tensors(self) -> dict[str, TensorSpec]:
        H, qd = self.heads, self.dim + self.rot_dim
        specs = {"q": TensorSpec((H * qd, self.hidden)), "dkv": TensorSpec((self.kv_rank + self.rot_dim, self.hidden)),
                 "dkv.norm": TensorSpec((self.kv_rank,), "vector"), "uk": TensorSpec((H * self.dim, self.kv_rank)),
                 "uv": TensorSpec((H * self.vdim, self.kv_rank)), "o": TensorSpec((self.hidden, H * self.vdim))}
        if self.sink:
            specs["sink"] = TensorSpec((H,), "vector")
        if self.gated:
            specs["g"] = TensorSpec((H, self.hidden))
        return specs

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.position.load({}, runtime)
        H, qd = self.heads, self.dim + self.rot_dim
        # One operand [q | down | gate] (rows padded to a multiple of 8).
        rows = [tensors["q"], tensors["dkv"]]
        self.down_col = H * qd
        self.gate_col = self.down_col + self.kv_rank + self.rot_dim
        total = self.gate_col
        if self.gated:
            rows.append(tensors["g"])
            total += H
        if total % 8:
            rows.append(torch.zeros(8 - total % 8, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        self.in_proj = torch.cat(rows, dim=0).contiguous()
        self.down_norm = tensors["dkv.norm"].contiguous()
        self.uk = tensors["uk"].view(H, self.dim, self.kv_rank).contiguous()  # q_lat = q_plain @ uk_h
        self.uv_t = tensors["uv"].view(H, self.vdim, self.kv_rank).transpose(1, 2).contiguous()  # [H, rank, vdim]
        self.o = tensors["o"].contiguous()
        self.sink_logits = tensors["sink"].contiguous() if self.sink else None

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        if ctx.kv is None:
            raise RuntimeError("an attention mixer needs cache pages")
        H, qd, step = self.heads, self.dim + self.rot_dim, ctx.step
        proj = ops.linear(h, self.in_proj)
        tokens = proj.shape[0]
        ops.latent_prepare(proj, 0, H, qd, self.down_col, self.kv_rank, self.rot_dim, self.down_norm, self.norm_eps,
                           self.position.table(), step.positions, ctx.kv)
        q = proj[:, : H * qd].view(tokens, H, qd)
        q_lat = ops.batched_mm(q[:, :, : self.dim].transpose(0, 1), self.uk)  # [H, tokens, rank]
        o_lat = torch.empty(H, tokens, self.kv_rank, dtype=proj.dtype, device=proj.device)
        ops.latent_attention(q_lat, q[:, :, self.dim:], ctx.kv, step, self.scale, self.sink_logits,
                             proj[:, self.gate_col:] if self.gated else None, o_lat)
        out = torch.empty(tokens, H, self.vdim, dtype=proj.dtype, device=proj.device)
        ops.batched_mm(o_lat, self.uv_t, out=out.transpose(0, 1))
        return ops.linear(out.view(tokens, H * self.vdim), self.o)


@register_mixer("sink_window_attention")
class SinkWindowAttention(Mixer):
    """Grouped-query causal attention with the options a sliding-window design with a softmax sink
    needs, each a parameter:

    hidden, heads, kv_heads: sizes; dim: width of a query/key head; vdim: width of a value head
    scale:      multiplies q.k
    window:     None, or how many latest positions (the query's own included) are visible;
    keep_first: with a window, how many of the request's first positions stay visible behind it
                (they keep their own positions for the rotation)
    norm_eps:   None, or the eps of an RMS norm of every q and k head, with a weight of the head's size
                shared by the heads (tensors `q.norm`, `k.norm`), applied before the rotation;
    norm_weight: False for that norm without weights (no such tensors)
    position:   PartSpec of a half-split rotary encoding over the first `dims` <= dim of a head
    bias:       q, k and v projections have biases (`q.b`, `k.b`, `v.b`), added before the norm
    sink:       True: the softmax's denominator also holds exp(sink_h), one learned number a head
                (`sink`), unscaled, with no key and no value; "zero": the same with every sink_h = 0 and no
                tensor, i.e. a one added to the denominator
    values:     "own": a value projection `v`; "keys": there is none, and the values are the projected
                keys as the product leaves them, ahead of the norm and the rotation (no biases; vdim = dim)
    own_kv:     False for a layer without k/v tensors that reads another layer's cache (as that cache
                holds the keys: normed and rotated) with queries, window and sink of its own
    norm_over:  "head": the norm above, every head by itself; "projection": one root mean square over
                all of a token's query heads at once (and one over all its key heads), the weights
                `q.norm` [heads * dim] and `k.norm` [kv_heads * dim] of the whole projection's size
    gated:      the heads' outputs are multiplied element by element by sigmoid(g h) (`g`
                [heads * vdim, hidden]) ahead of the output projection; g reads the mixer's own input
    chunk:      None, or the length of the runs that positions are cut into (from the request's
                position 0): a query sees key j <= i only of its own run
    softcap:    None, or c: a scaled score s becomes c tanh(s / c) ahead of the softmax
    The position part may pair dims half-split (i, i + dims / 2) or interleaved (2i, 2i + 1).

    Tensors: `q` [heads * dim, hidden], `k` [kv_heads * dim, hidden], `v` [kv_heads * vdim, hidden],
    `o` [hidden, heads * vdim]."""

    graph_safe = True
    graph_safe_mixed = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 window: int | None = None, keep_first: int = 0, norm_eps: float | None = None,
                 position: PartSpec | None = None, bias: bool = False, sink: bool = False, own_kv: bool = True,
                 norm_over: str = "head", gated: bool = False, chunk: int | None = None,
                 softcap: float | None = None, norm_weight: bool = True, values: str = "own") -> None:
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads do not divide into {kv_heads} groups")
        if dim > 256 or vdim > 256:
            raise ValueError(f"head widths of at most 256, got {dim} and {vdim}")
        if keep_first and window is None:
            keep_first = 0  # everything is visible anyway
        if norm_over not in ("head", "projection"):
            raise ValueError(f"norm_over is 'head' or 'projection', not {norm_over!r}")
        if chunk is not None and (chunk < 1 or keep_first):
            raise ValueError("chunk is a positive number of positions, and keeps no first positions")
        if softcap is not None and softcap <= 0:
            raise ValueError(f"softcap must be positive, got {softcap}")
        if sink not in (False, True, "zero"):
            raise ValueError(f"sink is False, True or 'zero', not {sink!r}")
        if values not in ("own", "keys") or (values == "keys" and (vdim != dim or bias)):
            raise ValueError("values are 'own' or, without biases and with vdim = dim, 'keys'")
        self.norm_weight, self.values = bool(norm_weight), values
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = hidden, heads, kv_heads, dim, vdim
        self.scale, self.window, self.keep_first, self.norm_eps = float(scale), window, int(keep_first), norm_eps
        self.bias, self.sink, self.own_kv = bias, sink, own_kv
        self.norm_over, self.gated, self.chunk, self.softcap = norm_over, gated, chunk, softcap
        self.position = POSITIONS.build(position or PartSpec("none"))
        self.interleaved = getattr(self.position, "pairing", "half") == "interleaved"
        if getattr(self.position, "dims", 0) > dim:
            raise ValueError(f"{self.position.dims} rotary dims do not fit a head of {dim}")

    def kv_spec(self) -> KVSpec:
        return KVSpec(((self.kv_heads, self.dim), (self.kv_heads, self.vdim)), self.window, keep_first=self.keep_first,
                      chunk=self.chunk)

    def tensors(self) -> dict[str, TensorSpec]:
        H, G, dk, dv = self.heads, self.kv_heads, self.dim, self.vdim
        specs = {"q": TensorSpec((H * dk, self.hidden)), "o": TensorSpec((self.hidden, H * dv))}
        if self.bias:
            specs["q.b"] = TensorSpec((H * dk,))
        whole = self.norm_over == "projection"
        if self.norm_eps is not None and self.norm_weight:
            specs["q.norm"] = TensorSpec((H * dk if whole else dk,), "vector")
        if self.sink is True:
            specs["sink"] = TensorSpec((H,), "vector")
        if self.gated:
            specs["g"] = TensorSpec((H * dv, self.hidden))
        if self.own_kv:
            specs["k"] = TensorSpec((G * dk, self.hidden))
            if self.values == "own":
                specs["v"] = TensorSpec((G * dv, self.hidden))
            if self.bias:
                specs["k.b"], specs["v.b"] = TensorSpec((G * dk,)), TensorSpec((G * dv,))
            if self.norm_eps is not None and self.norm_weight:
                specs["k.norm"] = TensorSpec((G * dk if whole else dk,), "vector")
        return specs

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.position.load({}, runtime)
        names = (["q", "k", "v"] if self.values == "own" else ["q", "k"]) if self.own_kv else ["q"]
        if self.gated:
            names.append("g")  # last, so that the columns of q, k and v stay where they are without it
        rows = [tensors[name] for name in names]
        self.k_col = self.heads * self.dim
        # Values that are the keys are read from the keys' columns of the projected rows.
        self.v_col = self.k_col + (self.kv_heads * self.dim if self.values == "own" else 0)
        self.gate_col = self.k_col + sum(r.shape[0] for r in rows[1:len(names) - int(self.gated)])
        total = sum(r.shape[0] for r in rows)
        pad = -total % 8  # rows of the operand in steps of 8, for the kernels that want them so
        if pad:
            rows.append(torch.zeros(pad, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        self.in_proj = torch.cat(rows, dim=0).contiguous()
        self.in_bias = None
        if self.bias:
            parts = [tensors[name + ".b"] if name != "g" else torch.zeros(tensors["g"].shape[0], dtype=rows[0].dtype,
                                                                          device=rows[0].device) for name in names]
            if pad:
                parts.append(torch.zeros(pad, dtype=parts[0].dtype, device=parts[0].device))
            self.in_bias = torch.cat(parts).contiguous()
        weighted = self.norm_eps is not None and self.norm_weight
        self.q_norm = tensors["q.norm"].contiguous() if weighted else None
        self.k_norm = tensors["k.norm"].contiguous() if weighted and self.own_kv else None
        self.sink_logits = None
        if self.sink is True:
            self.sink_logits = tensors["sink"].contiguous()
        elif self.sink == "zero":
            self.sink_logits = torch.zeros(self.heads, dtype=torch.float32, device=runtime.device)
        self.o = tensors["o"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return ops.linear(self.forward_heads(ops.linear(h, self.in_proj), 0, ctx), self.o)

    def forward_heads(self, proj: torch.Tensor, col0: int, ctx) -> torch.Tensor:
        """The heads' outputs side by side, ahead of the output projection, from projected rows whose
        columns from `col0` on are this mixer's input projection (a mixer that runs several side by side
        makes their input projections in one product)."""
        if ctx.kv is None:
            raise RuntimeError("an attention mixer needs cache pages")
        if ctx.kv.writes and not self.own_kv:
            raise RuntimeError("a mixer without k/v projections cannot own a cache entry")
        if col0 and self.in_bias is not None:
            raise RuntimeError("biased projections start at the projected rows' first column")
        q = ops.qkv_prepare(proj, col0, col0 + self.k_col, col0 + self.v_col, self.heads, self.dim, self.in_bias, self.q_norm,
                            self.k_norm, self.norm_eps, self.position.table(), ctx.step.positions, ctx.kv,
                            store=self.own_kv, whole=self.norm_over == "projection", interleaved=self.interleaved)
        return ops.paged_attention(q, ctx.kv, ctx.step, self.scale, gate=proj if self.gated else None,
                                   gate_col=col0 + self.gate_col, sink=self.sink_logits, window=self.window,
                                   keep_first=self.keep_first, chunk=self.chunk, softcap=self.softcap)
