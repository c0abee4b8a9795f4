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
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import Mixer, StateSpec, TensorSpec, register_mixer


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
