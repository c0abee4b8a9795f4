"""Feed-forward parts.

Reference: SwiGLU with gate and up fused on the output axis at load
(src/mlx_omnia/engine/core/layers.py:253-272, src/mlx_omnia/engine/checkpoint.py:333-347).
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """down(silu(gate(h)) * up(h)), no biases.

    hidden, inner: widths. The checkpoint's `gate_proj` and `up_proj` are stacked into
    one [2 * inner, hidden] operand at load so the step runs one product for both.
    """

    takes_pending = True

    def __init__(self, hidden: int, inner: int) -> None:
        self.hidden, self.inner = hidden, inner

    def tensors(self) -> dict[str, TensorSpec]:
        return {
            "gate_proj.weight": TensorSpec((self.inner, self.hidden)),
            "up_proj.weight": TensorSpec((self.inner, self.hidden)),
            "down_proj.weight": TensorSpec((self.hidden, self.inner)),
        }

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return ops.linear(ops.linear_swiglu(h, self.gate_up), self.down)


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    """down(act(up(h))), no biases and no gate.

    hidden, inner: widths; activation: "relu2" (the square of relu), "gelu_tanh" or "silu".
    Tensors: `up` [inner, hidden], `down` [hidden, inner].
    """

    def __init__(self, hidden: int, inner: int, activation: str = "relu2") -> None:
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"dense_mlp activation {activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.hidden, self.inner, self.activation = hidden, inner, activation

    def tensors(self) -> dict[str, TensorSpec]:
        return {"up": TensorSpec((self.inner, self.hidden)), "down": TensorSpec((self.hidden, self.inner))}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.up, self.down = tensors["up"].contiguous(), tensors["down"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return ops.linear(ops.linear_act(h, self.up, self.activation), self.down)


@register_feed_forward("clamped_glu_mlp")
class ClampedGLUMLP(FeedForward):
    """down(g * sigmoid(alpha * g) * (u + 1)) with g = min(gate(h), limit) and
    u = clamp(up(h), -limit, limit); no biases.

    hidden, inner: widths; limit: the clamp; alpha: the sigmoid's slope.
    Tensors: `gate`, `up` [inner, hidden] (stacked into one operand at load), `down` [hidden, inner].
    """

    def __init__(self, hidden: int, inner: int, limit: float, alpha: float = 1.702) -> None:
        if limit <= 0:
            raise ValueError(f"clamped_glu_mlp needs a positive limit, got {limit}")
        self.hidden, self.inner, self.limit, self.alpha = hidden, inner, float(limit), float(alpha)

    def tensors(self) -> dict[str, TensorSpec]:
        return {"gate": TensorSpec((self.inner, self.hidden)), "up": TensorSpec((self.inner, self.hidden)),
                "down": TensorSpec((self.hidden, self.inner))}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.down = tensors["down"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return ops.linear(ops.linear_clamped_glu(h, self.gate_up, self.alpha, self.limit), self.down)


@register_feed_forward("relu_glu_mlp")
class ReluGLUMLP(FeedForward):
    """down(relu(gate(h)) * up(h)), no biases.

    hidden, inner: widths. Tensors: `gate`, `up` [inner, hidden] (stacked into one operand at load),
    `down` [hidden, inner].
    """

    def __init__(self, hidden: int, inner: int) -> None:
        self.hidden, self.inner = hidden, inner

    def tensors(self) -> dict[str, TensorSpec]:
        return {"gate": TensorSpec((self.inner, self.hidden)), "up": TensorSpec((self.inner, self.hidden)),
                "down": TensorSpec((self.hidden, self.inner))}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.down = tensors["down"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return ops.linear(ops.linear_relu_glu(h, self.gate_up), self.down)


@register_feed_forward("table_experts")
class TableExperts(FeedForward):
    """A mixture of `experts` small clamped gated units of which every token uses `top`, chosen by
    no router: row `token id` of an integer table names the token's experts (the entries of a row
    differ), and each of them weighs 1 / top.

    hidden, inner: widths of an expert; vocab: rows of the table; limit, alpha: an expert is
    down(g sigmoid(alpha g) (u + 1)) with g = min(gate h, limit), u = clamp(up h, -limit, limit).
    Tensors: `table` [vocab, top] (integers), and per expert i `e<i>.gate`, `e<i>.up` [inner, hidden],
    `e<i>.down` [hidden, inner] (stacked at load).
    """

    def __init__(self, hidden: int, inner: int, experts: int, top: int, vocab: int, limit: float,
                 alpha: float = 1.702) -> None:
        if experts < 1 or not 1 <= top <= experts:
            raise ValueError(f"table_experts of {experts} experts, {top} a token")
        if limit <= 0:
            raise ValueError(f"table_experts needs a positive limit, got {limit}")
        self.hidden, self.inner, self.experts, self.top, self.vocab = hidden, inner, experts, top, vocab
        self.limit, self.alpha = float(limit), float(alpha)

    def tensors(self) -> dict[str, TensorSpec]:
        specs = {"table": TensorSpec((self.vocab, self.top), "table_i32")}
        for e in range(self.experts):
            specs[f"e{e}.gate"] = TensorSpec((self.inner, self.hidden))
            specs[f"e{e}.up"] = TensorSpec((self.inner, self.hidden))
            specs[f"e{e}.down"] = TensorSpec((self.hidden, self.inner))
        return specs

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.table = tensors["table"].contiguous()
        self.gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0)
                                    for e in range(self.experts)]).contiguous()
        self.down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return ops.moe_experts(h, None, None, self.gate_up, self.down, self.top, ctx.step, table=self.table,
                               token_ids=ctx.step.token_ids, alpha=self.alpha, limit=self.limit)


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of `experts` small gated feed-forward layers of which every token uses `top`.

    hidden, inner: widths of an expert (down(silu(gate h) * (up h)), no biases)
    experts:  experts with tensors; identity: router outputs beyond them whose expert hands its
              input back; top: choices per token
    The router's logits are taken in float32 (its matrix is kept in float32 whatever the engine's
    dtype), the scores are a softmax over all experts + identity outputs; the choice is by score +
    `correction`, the weight is the score itself, not renormalised.
    scoring:  "softmax" (above) or "sigmoid": every output's score is its own sigmoid
    weigh:    "output": y = sum of score * expert(h); "input": y = sum of expert(score * h), the chosen
              expert is given the token multiplied by its score and its output counts as it is
    shared_inner: None, or the inner width of one more gated expert (`shared.gate`, `shared.up`,
              `shared.down`) that every token uses unweighted and whose output is added
    Tensors: `router` [experts + identity, hidden], `correction` [experts + identity], and per expert i
    `e<i>.gate`, `e<i>.up` [inner, hidden], `e<i>.down` [hidden, inner] (stacked at load).
    """

    def __init__(self, hidden: int, inner: int, experts: int, top: int, identity: int = 0,
                 correction: bool = True, scoring: str = "softmax", weigh: str = "output",
                 shared_inner: int | None = None) -> None:
        if experts < 1 or identity < 0 or not 1 <= top <= experts + identity:
            raise ValueError(f"routed_experts of {experts} experts and {identity} identity ones, {top} a token")
        if scoring not in ("softmax", "sigmoid") or weigh not in ("output", "input"):
            raise ValueError(f"routed_experts scoring {scoring!r}, weigh {weigh!r}")
        self.hidden, self.inner, self.experts, self.identity, self.top = hidden, inner, experts, identity, top
        self.corrected, self.scoring, self.weigh, self.shared_inner = correction, scoring, weigh, shared_inner

    def tensors(self) -> dict[str, TensorSpec]:
        outputs = self.experts + self.identity
        specs = {"router": TensorSpec((outputs, self.hidden), "vector")}
        if self.corrected:
            specs["correction"] = TensorSpec((outputs,), "vector")
        for e in range(self.experts):
            specs[f"e{e}.gate"] = TensorSpec((self.inner, self.hidden))
            specs[f"e{e}.up"] = TensorSpec((self.inner, self.hidden))
            specs[f"e{e}.down"] = TensorSpec((self.hidden, self.inner))
        if self.shared_inner is not None:
            specs["shared.gate"] = TensorSpec((self.shared_inner, self.hidden))
            specs["shared.up"] = TensorSpec((self.shared_inner, self.hidden))
            specs["shared.down"] = TensorSpec((self.hidden, self.shared_inner))
        return specs

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.router = tensors["router"].contiguous()
        self.correction = tensors["correction"].contiguous() if self.corrected else None
        self.gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0)
                                    for e in range(self.experts)]).contiguous()
        self.down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).contiguous()
        self.shared_gate_up = self.shared_down = None
        if self.shared_inner is not None:
            self.shared_gate_up = torch.cat([tensors["shared.gate"], tensors["shared.up"]], dim=0).contiguous()
            self.shared_down = tensors["shared.down"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        extra = None
        if self.shared_gate_up is not None:
            extra = ops.linear(ops.linear_swiglu(h, self.shared_gate_up), self.shared_down)
        return ops.moe_experts(h, self.router, self.correction, self.gate_up, self.down, self.top, ctx.step,
                               scoring=self.scoring, weigh=self.weigh, extra=extra)
