"""Recurrent mixers: a fixed-size state per request instead of a cache that grows.

`channel_delta` is a gated delta rule whose decay is per head and key channel. With S a head's
state [dim, vdim], per token: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q (the
read-out sees the token's own write). q, k and v come through a short causal convolution and SiLU;
q and k are unit vectors per head (q also times dim^-1/2); g = exp(-exp(A_log) softplus(low-rank(h) +
dt_bias)); beta = sigmoid(b(h)); o is RMS-normed per head, weighted, gated by sigmoid(low-rank(h)),
and projected out.

`decay_attention` is linear attention with one constant decay per head: per head S <- decay_h S +
k v^T and o = S^T q with q, k and v behind SiLU and no other scale; the heads' outputs side by side
are RMS-normed together, weighted, gated by sigmoid(g(h)), and projected out.

`gated_state_attention` is linear attention whose decay is a constant per head or a factor per token
and key channel that the token sets through a low-rank map: S <- diag(a) S + k v^T, o = S^T q, with q
and k optionally rotated and scaled in float32, every head's o divided by its own root mean square,
and a silu or sigmoid gate.

`gated_channel_recurrence` is a recurrent block with one number of state a channel: a short causal
convolution, gates that are sigmoids of block-diagonal maps, S <- a S + sqrt(1 - a^2) i u with
a = exp(-c r softplus(lam)), the output multiplied by a tanh-GELU branch.

`side_by_side` runs two mixers on the same input and adds their outputs with a constant each.
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import MIXERS, POSITIONS, LayerContext, Mixer, PartSpec, StateSpec, TensorSpec, register_mixer


@register_mixer("channel_delta")
class ChannelDelta(Mixer):
    """hidden: model width; heads value heads of `vdim`; kv_heads query/key heads of `dim` (value head
    h reads query/key head h // (heads / kv_heads)); conv: taps of the short convolution;
    decay_rank, gate_rank: inner widths of the two low-rank maps; norm_eps: eps of the output norm;
    unit_eps: eps under the root of the unit norms.

    Tensors: q, k [kv_heads * dim, hidden]; v [heads * vdim, hidden]; q.conv, k.conv, v.conv
    [channels, taps] (last column: the current token); b [heads, hidden]; a1 [decay_rank, hidden],
    a2 [heads * dim, decay_rank], dt_bias [heads * dim], A_log [heads]; g1 [gate_rank, hidden],
    g2 [heads * vdim, gate_rank]; norm [vdim]; o [hidden, heads * vdim].
    State (float32): S [heads, dim, vdim] and the convolution's last taps - 1 inputs."""

    graph_safe = True
    graph_safe_mixed = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, decay_rank: int,
                 gate_rank: int, norm_eps: float, unit_eps: float = 1e-6) -> None:
        if heads % kv_heads:
            raise ValueError(f"{heads} value heads do not divide into {kv_heads} query/key heads")
        if not 1 <= conv <= ops.MAX_CONV_TAPS:
            raise ValueError(f"a short convolution of {conv} taps (1 to {ops.MAX_CONV_TAPS})")
        if vdim > 1024:
            raise ValueError("channel_delta takes value heads of at most 1024")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim, self.conv = hidden, heads, kv_heads, dim, vdim, conv
        self.decay_rank, self.gate_rank, self.norm_eps, self.unit_eps = decay_rank, gate_rank, float(norm_eps), unit_eps
        self.channels = 2 * kv_heads * dim + heads * vdim

    def state_spec(self):
        return {"S": StateSpec((self.heads, self.dim, self.vdim), torch.float32),
                "conv": StateSpec((self.conv - 1, self.channels), torch.float32)}

    def tensors(self) -> dict[str, TensorSpec]:
        qk, v, d = self.kv_heads * self.dim, self.heads * self.vdim, self.hidden
        return {
            "q": TensorSpec((qk, d)), "k": TensorSpec((qk, d)), "v": TensorSpec((v, d)),
            "q.conv": TensorSpec((qk, self.conv), "vector"), "k.conv": TensorSpec((qk, self.conv), "vector"),
            "v.conv": TensorSpec((v, self.conv), "vector"),
            "b": TensorSpec((self.heads, d)), "A_log": TensorSpec((self.heads,), "vector"),
            "a1": TensorSpec((self.decay_rank, d)), "a2": TensorSpec((self.heads * self.dim, self.decay_rank)),
            "dt_bias": TensorSpec((self.heads * self.dim,), "vector"),
            "g1": TensorSpec((self.gate_rank, d)), "g2": TensorSpec((v, self.gate_rank)),
            "norm": TensorSpec((self.vdim,), "vector"), "o": TensorSpec((d, v)),
        }

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        # One operand [q | k | v | b | a1 | g1] (rows padded to a multiple of 8), so the step runs a
        # single input projection; the convolution's taps side by side in the same channel order.
        rows = [tensors[name] for name in ("q", "k", "v", "b", "a1", "g1")]
        self.beta_col = self.channels
        self.a1_col = self.beta_col + self.heads
        self.g1_col = self.a1_col + self.decay_rank
        total = self.g1_col + self.gate_rank
        if total % 8:
            rows.append(torch.zeros(8 - total % 8, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        self.in_proj = torch.cat(rows, dim=0).contiguous()
        self.taps = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0).contiguous()
        # The second halves of the two low-rank maps as one block-diagonal operand: [a1 | g1] of the
        # projected rows goes in, [decay logits | gate logits] comes out (the zeros add nothing).
        a2, g2 = tensors["a2"], tensors["g2"]
        self.second = torch.zeros(a2.shape[0] + g2.shape[0], self.decay_rank + self.gate_rank, dtype=a2.dtype,
                                  device=a2.device)
        self.second[: a2.shape[0], : self.decay_rank] = a2
        self.second[a2.shape[0]:, self.decay_rank:] = g2
        self.o = tensors["o"].contiguous()
        self.A_log, self.dt_bias = tensors["A_log"].contiguous(), tensors["dt_bias"].contiguous()
        self.norm_weight = tensors["norm"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        step, state = ctx.step, ctx.state
        proj = ops.linear(h, self.in_proj)
        qk = self.kv_heads * self.dim
        both = ops.linear(proj[:, self.a1_col: self.g1_col + self.gate_rank], self.second)
        decay, gate = both[:, : self.heads * self.dim], both[:, self.heads * self.dim:]
        conv = ops.short_conv(proj, 0, self.channels, self.taps, state["conv"], step, 2 * qk, self.dim, self.unit_eps,
                              qk, self.dim ** -0.5, decay, self.A_log, self.dt_bias, self.beta_col, self.heads)
        out = ops.delta_rule(conv, self.channels, self.kv_heads, self.heads, self.dim, self.vdim, proj, 0, gate,
                             self.norm_weight, self.norm_eps, state["S"], state["conv"], self.conv, step)
        return ops.linear(out, self.o)


@register_mixer("decay_attention")
class DecayAttention(Mixer):
    """hidden: model width; heads of `dim` (queries and keys) and `vdim` (values); decay: one constant
    in (0, 1] per head; norm_eps: eps of the output norm.

    Tensors: q, k [heads * dim, hidden]; v, g [heads * vdim, hidden]; norm [heads * vdim];
    o [hidden, heads * vdim].
    State (float32): S [heads, dim, vdim], zeros at a request's start."""

    graph_safe = True
    graph_safe_mixed = True
    takes_pending = True  # h goes to the in-projection and nowhere else

    def __init__(self, hidden: int, heads: int, dim: int, vdim: int, decay: tuple[float, ...], norm_eps: float) -> None:
        decay = tuple(float(d) for d in decay)
        if len(decay) != heads:
            raise ValueError(f"decay_attention of {heads} heads was given {len(decay)} decays")
        if dim < 1 or dim > 256 or vdim < 1:
            raise ValueError(f"decay_attention takes keys of 1 to 256 and values of at least 1, got {dim} and {vdim}")
        self.hidden, self.heads, self.dim, self.vdim, self.decay, self.norm_eps = hidden, heads, dim, vdim, decay, float(norm_eps)

    def state_spec(self):
        return StateSpec((self.heads, self.dim, self.vdim), torch.float32)

    def tensors(self) -> dict[str, TensorSpec]:
        qk, v, d = self.heads * self.dim, self.heads * self.vdim, self.hidden
        return {"q": TensorSpec((qk, d)), "k": TensorSpec((qk, d)), "v": TensorSpec((v, d)), "g": TensorSpec((v, d)),
                "norm": TensorSpec((v,), "vector"), "o": TensorSpec((d, v))}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        # One operand [q | k | v | g] (rows padded to a multiple of 8): a single input projection.
        rows = [tensors[name] for name in ("q", "k", "v", "g")]
        qk, v = self.heads * self.dim, self.heads * self.vdim
        self.k_col, self.v_col, self.gate_col = qk, 2 * qk, 2 * qk + v
        total = self.gate_col + v
        if total % 8:
            rows.append(torch.zeros(8 - total % 8, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        self.in_proj = torch.cat(rows, dim=0).contiguous()
        self.norm_weight = tensors["norm"].contiguous()
        self.o = tensors["o"].contiguous()
        self.decays = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def forward(self, h, ctx) -> torch.Tensor:
        proj = ops.linear(h, self.in_proj)
        out = ops.lightning_attention(proj, 0, self.k_col, self.v_col, self.gate_col, self.heads, self.dim, self.vdim,
                                      self.decays, self.norm_weight, self.norm_eps, ctx.state, ctx.step)
        return ops.linear(out, self.o)


@register_mixer("gated_state_attention")
class GatedStateAttention(Mixer):
    """hidden: model width; heads of `dim` (queries and keys) and `vdim` (values); norm_eps: eps under
    the root of the heads' output norms.
    decay:      a constant in (0, 1] per head, or None for a decay per token and key channel,
                a = sigmoid(a2 (a1 h) + a2.b)^(1 / tau), with `decay_rank` the inner width of the map
    position:   None, or the PartSpec of a half-split rotary encoding applied to q and k (float32)
    q_scale, k_scale: multiply q and k after the rotation (float32)
    norm_weight: the heads' output norm has a weight `norm` [vdim] that the heads share
    gate:       "silu" or "sigmoid" of g h, multiplied into the normed outputs

    Tensors: q, k [heads * dim, hidden]; v, g [heads * vdim, hidden]; o [hidden, heads * vdim];
    norm [vdim]; a1 [decay_rank, hidden], a2 [heads * dim, decay_rank], a2.b [heads * dim].
    State (float32): S [heads, dim, vdim], zeros at a request's start."""

    graph_safe = True
    graph_safe_mixed = True

    def __init__(self, hidden: int, heads: int, dim: int, vdim: int, norm_eps: float,
                 decay: tuple[float, ...] | None = None, decay_rank: int = 0, tau: float = 1.0,
                 position: PartSpec | None = None, q_scale: float = 1.0, k_scale: float = 1.0,
                 norm_weight: bool = True, gate: str = "silu") -> None:
        if decay is not None:
            decay = tuple(float(d) for d in decay)
            if len(decay) != heads:
                raise ValueError(f"gated_state_attention of {heads} heads was given {len(decay)} decays")
        elif decay_rank < 1 or tau <= 0:
            raise ValueError("a decay per channel needs the inner width of its map and a positive tau")
        if dim < 1 or dim > 256 or vdim < 1:
            raise ValueError(f"gated_state_attention takes keys of 1 to 256 and values of at least 1, got {dim} and {vdim}")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"the gate is 'silu' or 'sigmoid', not {gate!r}")
        self.hidden, self.heads, self.dim, self.vdim, self.norm_eps = hidden, heads, dim, vdim, float(norm_eps)
        self.decay, self.decay_rank, self.tau = decay, int(decay_rank), float(tau)
        self.q_scale, self.k_scale, self.norm_weight, self.gate = float(q_scale), float(k_scale), bool(norm_weight), gate
        self.position = POSITIONS.build(position or PartSpec("none"))
        if getattr(self.position, "pairing", "half") != "half":
            raise ValueError("gated_state_attention rotates half-split pairs")
        if getattr(self.position, "dims", 0) > dim:
            raise ValueError(f"{self.position.dims} rotary dims do not fit a head of {dim}")

    def state_spec(self):
        return StateSpec((self.heads, self.dim, self.vdim), torch.float32)

    def tensors(self) -> dict[str, TensorSpec]:
        qk, v, d = self.heads * self.dim, self.heads * self.vdim, self.hidden
        specs = {"q": TensorSpec((qk, d)), "k": TensorSpec((qk, d)), "v": TensorSpec((v, d)), "g": TensorSpec((v, d)),
                 "o": TensorSpec((d, v))}
        if self.norm_weight:
            specs["norm"] = TensorSpec((self.vdim,), "vector")
        if self.decay is None:
            specs.update({"a1": TensorSpec((self.decay_rank, d)), "a2": TensorSpec((qk, self.decay_rank)),
                          "a2.b": TensorSpec((qk,), "vector")})
        return specs

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.position.load({}, runtime)
        # One operand [q | k | v | g | a1] (rows padded to a multiple of 8): a single input projection.
        names = ["q", "k", "v", "g"] + (["a1"] if self.decay is None else [])
        rows = [tensors[name] for name in names]
        qk, v = self.heads * self.dim, self.heads * self.vdim
        self.k_col, self.v_col, self.gate_col, self.a1_col = qk, 2 * qk, 2 * qk + v, 2 * qk + 2 * v
        total = sum(r.shape[0] for r in rows)
        if total % 8:
            rows.append(torch.zeros(8 - total % 8, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        self.in_proj = torch.cat(rows, dim=0).contiguous()
        self.norm = tensors["norm"].contiguous() if self.norm_weight else None
        self.o = tensors["o"].contiguous()
        self.decays = self.a2 = self.a2_bias = None
        if self.decay is not None:
            self.decays = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)
        else:
            # The map's second half in float32: its few inputs are the projected rows' (rounded as any
            # projection's), its outputs, the decays' logits, are not rounded on their way into the recurrence.
            self.a2, self.a2_bias = tensors["a2"].to(torch.float32).contiguous(), tensors["a2.b"].contiguous()

    def forward(self, h, ctx) -> torch.Tensor:
        return ops.linear(self.forward_heads(ops.linear(h, self.in_proj), 0, ctx), self.o)

    def forward_heads(self, proj: torch.Tensor, col0: int, ctx) -> torch.Tensor:
        """The heads' gated outputs side by side, ahead of the output projection, from projected rows
        whose columns from `col0` on are this mixer's input projection."""
        logits = None
        if self.decay is None:
            logits = ops.linear(proj[:, col0 + self.a1_col: col0 + self.a1_col + self.decay_rank].float(), self.a2)
        return ops.state_attention(proj, col0, col0 + self.k_col, col0 + self.v_col, col0 + self.gate_col, self.heads,
                                   self.dim, self.vdim, ctx.state, ctx.step, self.norm_eps, decay=self.decays,
                                   decay_logits=logits, decay_bias=self.a2_bias, tau=self.tau,
                                   inv_freq=self.position.table(), q_scale=self.q_scale, k_scale=self.k_scale,
                                   norm_weight=self.norm, gate=self.gate)


@register_mixer("gated_channel_recurrence")
class GatedChannelRecurrence(Mixer):
    """hidden: model width; width: channels of the recurrence, cut into `blocks` equal runs for the
    gates' block-diagonal maps; conv: taps of the causal convolution; c_decay: the constant c in
    a = exp(-c r softplus(lam)).

    Two branches read the input: y = gelu_tanh(y h + y.b) and u = conv(x h + x.b) (taps `conv`
    [width, taps], the last column the current token's, bias `conv.b`; zeros ahead of a request's
    start). Per run b of u: r = sigmoid(ra[b] u_b + ra.b[b]), i = sigmoid(ri[b] u_b + ri.b[b]) with
    ra[b], ri[b] square [out, in]. S <- a S + sqrt(1 - a^2) i u from S = 0; out = o (S * y).

    Tensors: x, y [width, hidden], x.b, y.b [width]; conv [width, taps], conv.b [width]; ra, ri
    [blocks, width / blocks, width / blocks], ra.b, ri.b [blocks, width / blocks]; lam [width];
    o [hidden, width].
    State (float32): S [width] and the convolution's last taps - 1 inputs."""

    graph_safe = True
    graph_safe_mixed = True

    def __init__(self, hidden: int, width: int, blocks: int, conv: int, c_decay: float = 8.0) -> None:
        if blocks < 1 or width % blocks:
            raise ValueError(f"{width} channels do not divide into {blocks} blocks")
        if not 1 <= conv <= ops.RGLRU_MAX_TAPS:
            raise ValueError(f"a convolution of {conv} taps (1 to {ops.RGLRU_MAX_TAPS})")
        self.hidden, self.width, self.blocks, self.conv, self.c_decay = hidden, width, blocks, conv, float(c_decay)

    def state_spec(self):
        return {"S": StateSpec((self.width,), torch.float32),
                "conv": StateSpec((max(self.conv - 1, 1), self.width), torch.float32)}

    def tensors(self) -> dict[str, TensorSpec]:
        w, d, b, bw = self.width, self.hidden, self.blocks, self.width // self.blocks
        return {"x": TensorSpec((w, d)), "y": TensorSpec((w, d)), "x.b": TensorSpec((w,), "vector"),
                "y.b": TensorSpec((w,), "vector"), "conv": TensorSpec((w, self.conv), "vector"),
                "conv.b": TensorSpec((w,), "vector"), "ra": TensorSpec((b, bw, bw), "vector"),
                "ri": TensorSpec((b, bw, bw), "vector"), "ra.b": TensorSpec((b, bw), "vector"),
                "ri.b": TensorSpec((b, bw), "vector"), "lam": TensorSpec((w,), "vector"), "o": TensorSpec((d, w))}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        rows = [tensors["x"], tensors["y"]]  # one operand [x | y]
        if 2 * self.width % 8:
            rows.append(torch.zeros(8 - 2 * self.width % 8, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        self.in_proj = torch.cat(rows, dim=0).contiguous()
        self.x_bias, self.y_bias = tensors["x.b"].contiguous(), tensors["y.b"].contiguous()
        self.taps, self.conv_bias = tensors["conv"].contiguous(), tensors["conv.b"].contiguous()
        # Both gates' maps side by side, input channels along the rows: [blocks, in, r's out | i's out], float32.
        self.gates = torch.cat([tensors["ra"].transpose(1, 2), tensors["ri"].transpose(1, 2)], dim=2).contiguous()
        self.r_bias, self.i_bias = tensors["ra.b"].reshape(-1).contiguous(), tensors["ri.b"].reshape(-1).contiguous()
        self.lam, self.o = tensors["lam"].contiguous(), tensors["o"].contiguous()

    takes_pending = True  # h goes to the in-projection and nowhere else

    def forward(self, h, ctx) -> torch.Tensor:
        return ops.linear(self.forward_heads(ops.linear(h, self.in_proj), 0, ctx), self.o)

    def forward_heads(self, proj: torch.Tensor, col0: int, ctx) -> torch.Tensor:
        """S * y for every channel, ahead of the output projection, from projected rows whose columns
        from `col0` on are this mixer's input projection."""
        return ops.gated_channel_recurrence(proj, col0, col0 + self.width, self.x_bias, self.y_bias, self.taps,
                                            self.conv_bias, self.gates, self.r_bias, self.i_bias, self.lam, self.c_decay,
                                            ctx.state["S"], ctx.state["conv"], ctx.step)


@register_mixer("side_by_side")
class SideBySide(Mixer):
    """Two mixers that read the same input; the result is left_scale * left(h) + right_scale * right(h),
    the sum taken in float32 and rounded once.

    left, right: PartSpecs of registered mixers; their tensors sit under `left.` and `right.`. At most
    one of the two may keep rows in the paged cache (the schedule entry's pages are that one's); each
    may keep per-request state, which this part hands to its owner.

    Two sides that each are an input projection `in_proj`, a `forward_heads(projected rows, first
    column, ctx)` and an output projection `o` run as one input product over both sides' stacked rows
    (so the mixer may take a pending residual step), and the left side's output product takes the
    right side's result and both constants in its epilogue; any other pair runs side by side as it is."""

    def __init__(self, left: PartSpec, right: PartSpec, left_scale: float = 1.0, right_scale: float = 1.0) -> None:
        self.sides = {"left": MIXERS.build(left), "right": MIXERS.build(right)}
        self.scales = {"left": float(left_scale), "right": float(right_scale)}
        if sum(side.kv_spec() is not None for side in self.sides.values()) > 1:
            raise ValueError("side_by_side takes at most one mixer that keeps rows in the paged cache")
        self.graph_safe = all(getattr(side, "graph_safe", False) for side in self.sides.values())
        self.graph_safe_mixed = all(getattr(side, "graph_safe_mixed", False) for side in self.sides.values())
        self._stateful = [name for name, side in self.sides.items() if side.state_spec() is not None]

    def kv_spec(self):
        return next((spec for spec in (side.kv_spec() for side in self.sides.values()) if spec is not None), None)

    def state_spec(self):
        if not self._stateful:
            return None
        if len(self._stateful) == 1:
            return self.sides[self._stateful[0]].state_spec()
        merged = {}
        for name in self._stateful:
            spec = self.sides[name].state_spec()
            for key, value in (spec.items() if isinstance(spec, dict) else [("", spec)]):
                merged[f"{name}.{key}" if key else name] = value
        return merged

    def initial_state(self):
        return self.sides[self._stateful[0]].initial_state() if len(self._stateful) == 1 else None

    def tensors(self) -> dict[str, TensorSpec]:
        return {f"{name}.{local}": spec for name, side in self.sides.items() for local, spec in side.tensors().items()}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        for name, side in self.sides.items():
            prefix = name + "."
            side.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, runtime)
        left, right = self.sides["left"], self.sides["right"]
        self.fused = all(hasattr(side, "forward_heads") and hasattr(side, "in_proj") and hasattr(side, "o")
                         and getattr(side, "in_bias", None) is None and side.in_proj.shape[0] % 8 == 0
                         for side in (left, right))
        self.takes_pending = self.fused  # h then goes to the one input product and nowhere else
        if self.fused:
            self.in_proj = torch.cat([left.in_proj, right.in_proj], dim=0).contiguous()
            self.right_col = left.in_proj.shape[0]
            left.in_proj, right.in_proj = self.in_proj[: self.right_col], self.in_proj[self.right_col:]

    def _context(self, name: str, ctx) -> LayerContext:
        side = self.sides[name]
        return LayerContext(ctx.step, ctx.kv if side.kv_spec() is not None else None, self._state_of(name, ctx.state),
                            ctx.entry, ctx.block_state, False)

    def _state_of(self, name: str, state):
        if name not in self._stateful:
            return None
        if len(self._stateful) == 1:
            return state
        if isinstance(self.sides[name].state_spec(), dict):
            prefix = name + "."
            return {k[len(prefix):]: v for k, v in state.items() if k.startswith(prefix)}
        return state[name]

    def forward(self, h, ctx) -> torch.Tensor:
        left, right = self.sides["left"], self.sides["right"]
        if not self.fused:
            outs = {name: side.forward(ops.settle(h), self._context(name, ctx)) for name, side in self.sides.items()}
            return ops.scaled_sum(outs["left"], self.scales["left"], outs["right"], self.scales["right"])
        proj = ops.linear(h, self.in_proj)
        mixed_right = ops.linear(right.forward_heads(proj, self.right_col, self._context("right", ctx)), right.o)
        return ops.linear_add(left.forward_heads(proj, 0, self._context("left", ctx)), left.o, self.scales["left"],
                              mixed_right, self.scales["right"])
