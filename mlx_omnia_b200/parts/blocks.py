"""Blocks: how a mixer, a feed-forward and norms sit around the residual stream.

The residual stream `x` is float32 [tokens, hidden] and is updated in place. A block
is handed `h`, its own entry norm already applied to `x` (the previous block's last
kernel produced it), and the norm that whatever runs next wants applied on the way
out, so each residual update is one fused pass: add the (normed) branch, then norm.
In a step of few rows that pass need not be a kernel of its own: where the part that
takes its result says `takes_pending`, the block hands it an `ops.PendingStep` instead
of `h`, the part's first product runs the step in front of itself, and the block then
picks up the new residual with `ops.residual_after`.

Reference: sandwich arrangement x + post(attn(input_ln(x))), then + post(mlp(pre_ff(.)))
(src/mlx_omnia/engine/models/muse_glimmer/layers/block.py:11-26).
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import (FEED_FORWARDS, MIXERS, NORMS, Block, Norm, PartSpec, StateSpec, TensorSpec,
                                       register_block)
from mlx_omnia_b200.parts.norms import RMSNorm


def residual_step(x: torch.Tensor, branch: torch.Tensor, branch_norm: Norm | None, out_norm: Norm | None,
                  may_pend: bool = False):
    """x += branch_norm(branch); return out_norm(x) (None without an out_norm).
    RMS norms take the fused kernel; any other norm class is applied by its own forward.
    With `may_pend` (whoever takes the result says it `takes_pending`) a step of few rows is
    not run here but handed on as an `ops.PendingStep`, for the taker's first product to run."""
    fused_b = branch_norm is None or (isinstance(branch_norm, RMSNorm) and branch_norm.groups == 1)
    fused_o = out_norm is None or (isinstance(out_norm, RMSNorm) and out_norm.groups == 1)
    if may_pend and fused_b and fused_o and out_norm is not None and ops.pending_supported(x, branch):
        return ops.PendingStep(x, branch, None if branch_norm is None else branch_norm.weight,
                               None if branch_norm is None else branch_norm.eps, out_norm.weight, out_norm.eps)
    if not fused_b:
        branch = branch_norm.forward(branch.float())
        branch_norm = None
    h = ops.add_rmsnorm(x, branch,
                        None if branch_norm is None else branch_norm.weight,
                        None if branch_norm is None else branch_norm.eps,
                        out_norm.weight if (fused_o and out_norm is not None) else None,
                        out_norm.eps if (fused_o and out_norm is not None) else None)
    if not fused_o:
        h = out_norm.forward(x)
    return h


class _TwoBranchBlock(Block):
    norm_names: tuple[str, ...] = ()

    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, norms: dict[str, PartSpec],
                 mixer_name: str = "self_attn", feed_forward_name: str = "mlp") -> None:
        missing = set(self.norm_names) - set(norms)
        if missing:
            raise ValueError(f"{type(self).__name__} needs the norms {sorted(missing)}")
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward)
        self.norms = {name: NORMS.build(norms[name]) for name in self.norm_names}
        self.mixer_name, self.feed_forward_name = mixer_name, feed_forward_name
        self.entry_norm = self.norms[self.norm_names[0]]

    def _mix(self, h, ctx):
        """The mixer's branch; `h` may be the block before's pending step, which a mixer that does
        not take such gets settled."""
        return self.mixer.forward(h if getattr(self.mixer, "takes_pending", False) else ops.settle(h), ctx)

    def children(self):
        yield self.mixer_name, self.mixer
        yield self.feed_forward_name, self.feed_forward
        yield from self.norms.items()

    def tensors(self) -> dict[str, TensorSpec]:
        return {f"{name}.{local}": spec for name, part in self.children() for local, spec in part.tensors().items()}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        for name, part in self.children():
            prefix = name + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, runtime)


@register_block("sandwich")
class SandwichBlock(_TwoBranchBlock):
    """Four norms: one before and one after each branch; the after-norm is on the branch."""

    norm_names = ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                  "post_feedforward_layernorm")

    def forward(self, x, h, ctx, exit_norm):
        n = self.norms
        a = self._mix(h, ctx)
        x = ops.residual_after(h, x)
        h2 = residual_step(x, a, n["post_attention_layernorm"], n["pre_feedforward_layernorm"],
                           getattr(self.feed_forward, "takes_pending", False))
        m = self.feed_forward.forward(h2, ctx)
        x = ops.residual_after(h2, x)
        return x, residual_step(x, m, n["post_feedforward_layernorm"], exit_norm, ctx.exit_may_pend)


@register_block("scaled_sandwich")
class ScaledSandwichBlock(Block):
    """A norm before and after each branch, the normed branch multiplied by a constant on its way
    into the residual: x += m * after(mixer(before(x))), then x += m * after2(ff(before2(x))). The
    feed-forward may be missing (the block then has one branch and two norms).

    mixer:        PartSpec of the mixer; feed_forward: PartSpec or None
    norms:        {"norm1", "norm1b"} and, with a feed-forward, {"norm2", "norm2b"}: the norm before
                  and the norm after (b) each branch
    branch_scale: m. It is folded into the after-norms' weights when they are loaded (one float32
                  product a weight), so the fused residual step needs no factor of its own; an
                  after-norm must therefore carry a weight.
    """

    def __init__(self, mixer: PartSpec, feed_forward: PartSpec | None, norms: dict[str, PartSpec],
                 branch_scale: float = 1.0, mixer_name: str = "mix", feed_forward_name: str = "mlp") -> None:
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward is not None else None
        wanted = ("norm1", "norm1b", "norm2", "norm2b") if feed_forward is not None else ("norm1", "norm1b")
        if set(wanted) - set(norms):
            raise ValueError(f"scaled_sandwich needs the norms {wanted}")
        self.norms = {name: NORMS.build(norms[name]) for name in wanted}
        self.branch_scale = float(branch_scale)
        self.mixer_name, self.feed_forward_name = mixer_name, feed_forward_name
        self.entry_norm = self.norms["norm1"]

    def children(self):
        yield self.mixer_name, self.mixer
        if self.feed_forward is not None:
            yield self.feed_forward_name, self.feed_forward
        yield from self.norms.items()

    def tensors(self) -> dict[str, TensorSpec]:
        return {f"{name}.{local}": spec for name, part in self.children() for local, spec in part.tensors().items()}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        for name, part in self.children():
            prefix = name + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, runtime)
        for name in ("norm1b", "norm2b"):
            norm = self.norms.get(name)
            if norm is None:
                continue
            if not isinstance(norm, RMSNorm) or norm.weight is None or norm.groups != 1:
                raise ValueError(f"scaled_sandwich's {name} must be an ungrouped rms_norm with a weight")
            if self.branch_scale != 1.0:
                norm.weight = (norm.weight * self.branch_scale).contiguous()

    def forward(self, x, h, ctx, exit_norm):
        n = self.norms
        a = self.mixer.forward(h if getattr(self.mixer, "takes_pending", False) else ops.settle(h), ctx)
        x = ops.residual_after(h, x)
        if self.feed_forward is None:
            return x, residual_step(x, a, n["norm1b"], exit_norm, ctx.exit_may_pend)
        h2 = residual_step(x, a, n["norm1b"], n["norm2"], getattr(self.feed_forward, "takes_pending", False))
        m = self.feed_forward.forward(h2, ctx)
        x = ops.residual_after(h2, x)
        return x, residual_step(x, m, n["norm2b"], exit_norm, ctx.exit_may_pend)


@register_block("pre_norm")
class PreNormBlock(_TwoBranchBlock):
    """Two norms, one before each branch; branches are added as they are."""

    norm_names = ("input_layernorm", "post_attention_layernorm")

    def forward(self, x, h, ctx, exit_norm):
        a = self._mix(h, ctx)
        x = ops.residual_after(h, x)
        h2 = residual_step(x, a, None, self.norms["post_attention_layernorm"],
                           getattr(self.feed_forward, "takes_pending", False))
        m = self.feed_forward.forward(h2, ctx)
        x = ops.residual_after(h2, x)
        return x, residual_step(x, m, None, exit_norm, ctx.exit_may_pend)


@register_block("hyper_pre_norm")
class HyperPreNormBlock(Block):
    """A pre-norm block whose residual may be several streams, whose mixer may read a token-shifted
    input, and whose feed-forward may be missing.

    hidden:       the model width
    mixer:        PartSpec of the mixer; feed_forward: PartSpec or None (the block then has one branch)
    norms:        {"norm1": spec, "norm2": spec} of `rms_norm` parts (grouped or not); norm2 only with
                  a feed-forward
    streams:      None for the ordinary residual x += branch. n >= 1 keeps n residual streams
                  x_1..x_n side by side ([tokens, n * hidden]); branch q (1 mixer, 2 feed-forward) reads
                  u = sum_s in_q[s] x_s and is written back as x_t = sum_s mix_q[s, t] x_s + out_q[t] y for
                  all t at once (tensors `hc<q>.in` [n], `hc<q>.out` [n], `hc<q>.mix` [n, n], from-stream
                  first). The embedding writes the n equal copies the streams start as.
    shift:        the mixer reads h + (h_before - h) * mu instead of its normed input h, with h_before
                  the normed input of the token before (zeros ahead of the first token) and mu the
                  tensor `shift` [hidden]; h_before of a request's last token is kept in a state slot.

    The block does its own entry (`entry_norm` is None). Given an exit norm (whatever follows is
    not a block of this kind: the model's final norm) it hands on the sum of the streams, normed."""

    entry_norm = None

    def __init__(self, hidden: int, mixer: PartSpec, feed_forward: PartSpec | None, norms: dict[str, PartSpec],
                 streams: int | None = None, shift: bool = False, mixer_name: str = "mix",
                 feed_forward_name: str = "mlp") -> None:
        if streams is not None and not 1 <= streams <= ops.MAX_STREAMS:
            raise ValueError(f"a residual of {streams} streams (at most {ops.MAX_STREAMS})")
        self.hidden, self.streams, self.shift = hidden, streams, shift
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward is not None else None
        wanted = ("norm1", "norm2") if feed_forward is not None else ("norm1",)
        if set(wanted) - set(norms):
            raise ValueError(f"hyper_pre_norm needs the norms {wanted}")
        self.norms = {name: NORMS.build(norms[name]) for name in wanted}
        for name, norm in self.norms.items():
            if not isinstance(norm, RMSNorm) or norm.convention == "none":
                raise ValueError(f"hyper_pre_norm's {name} must be an rms_norm with a weight")
        self.mixer_name, self.feed_forward_name = mixer_name, feed_forward_name

    def children(self):
        yield self.mixer_name, self.mixer
        if self.feed_forward is not None:
            yield self.feed_forward_name, self.feed_forward
        yield from self.norms.items()

    def branches(self) -> list[str]:
        return ["hc1", "hc2"] if self.feed_forward is not None else ["hc1"]

    def tensors(self) -> dict[str, TensorSpec]:
        specs = {f"{name}.{local}": spec for name, part in self.children() for local, spec in part.tensors().items()}
        if self.streams is not None:
            n = self.streams
            for hc in self.branches():
                specs.update({f"{hc}.in": TensorSpec((n,), "vector"), f"{hc}.out": TensorSpec((n,), "vector"),
                              f"{hc}.mix": TensorSpec((n, n), "vector")})
        if self.shift:
            specs["shift"] = TensorSpec((self.hidden,), "vector")
        return specs

    def state_spec(self):
        return {"shift": StateSpec((self.hidden,), torch.float32)} if self.shift else None

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        for name, part in self.children():
            prefix = name + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, runtime)
        self.hc = {hc: tuple(tensors[f"{hc}.{which}"].contiguous() for which in ("in", "mix", "out"))
                   if self.streams is not None else (None, None, None) for hc in self.branches()}
        self.mu = tensors["shift"].contiguous() if self.shift else None

    def forward(self, x, h, ctx, exit_norm):
        n = self.streams or 1
        if x.shape[1] != n * self.hidden:
            raise RuntimeError(f"a residual of {n} streams of {self.hidden} was handed {x.shape[1]} columns")
        dtype, step = self.runtime.dtype, ctx.step
        norm = self.norms["norm1"]
        a_in, a_mix, a_out = self.hc["hc1"]
        prev = last = None
        if self.shift:
            prev = ctx.block_state["shift"]
            last = torch.empty(step.num_seqs, self.hidden, dtype=torch.float32, device=x.device)
        h1 = ops.streams_enter(x, a_in, n, norm.weight, norm.eps, norm.groups, dtype, step, self.mu, prev, last)
        branch = self.mixer.forward(h1, ctx)
        if self.feed_forward is None:
            ops.streams_leave(x, branch, a_mix, a_out, n, step, last, prev)
        else:
            # Leaving the mixer's branch and entering the feed-forward's is one pass over the row.
            norm = self.norms["norm2"]
            b_in, b_mix, b_out = self.hc["hc2"]
            h2 = ops.streams_leave(x, branch, a_mix, a_out, n, step, last, prev,
                                   enter=(b_in, norm.weight, norm.eps, norm.groups))
            ops.streams_leave(x, self.feed_forward.forward(h2, ctx), b_mix, b_out, n)
        if exit_norm is None:
            return x, None
        if isinstance(exit_norm, RMSNorm) and exit_norm.convention != "none":
            total = torch.empty(x.shape[0], self.hidden, dtype=torch.float32, device=x.device)
            out = ops.streams_enter(x, None, n, exit_norm.weight, exit_norm.eps, exit_norm.groups, dtype, total=total)
            return total, out
        total = x.view(x.shape[0], n, self.hidden).sum(1) if n > 1 else x
        return total, exit_norm.forward(total)


@register_block("branch_norm")
class BranchNormBlock(Block):
    """Norms on the branches' outputs only: x += norm1(mixer(x)), then x += norm2(feed_forward(x)).
    Both branches read the residual itself (rounded to the engine's dtype), so the block has no entry
    norm; the rounding of the new residual for whoever reads it next is part of the residual step's
    one pass over the row. A block of this kind hands that rounded residual on, and takes it from
    the block before when that one made it.

    mixer:        PartSpec of the mixer; feed_forward: PartSpec or None (one branch only)
    norms:        {"norm1": spec, "norm2": spec} (norm2 only with a feed-forward)
    """

    entry_norm = None

    def __init__(self, mixer: PartSpec, feed_forward: PartSpec | None, norms: dict[str, PartSpec],
                 mixer_name: str = "mix", feed_forward_name: str = "mlp") -> None:
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward is not None else None
        wanted = ("norm1", "norm2") if feed_forward is not None else ("norm1",)
        if set(wanted) - set(norms):
            raise ValueError(f"branch_norm needs the norms {wanted}")
        self.norms = {name: NORMS.build(norms[name]) for name in wanted}
        self.mixer_name, self.feed_forward_name = mixer_name, feed_forward_name

    def children(self):
        yield self.mixer_name, self.mixer
        if self.feed_forward is not None:
            yield self.feed_forward_name, self.feed_forward
        yield from self.norms.items()

    def tensors(self) -> dict[str, TensorSpec]:
        return {f"{name}.{local}": spec for name, part in self.children() for local, spec in part.tensors().items()}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        for name, part in self.children():
            prefix = name + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, runtime)

    def _step(self, x, branch, norm, exit_norm, last: bool):
        """x += norm(branch); -> what the next reader wants: the exit norm's output after the block's
        last branch when one is asked for, else x rounded to the engine's dtype."""
        rms = isinstance(norm, RMSNorm) and norm.groups == 1
        if not rms:
            branch, norm = norm.forward(branch.float()).to(branch.dtype), None
        weight, eps = (norm.weight, norm.eps) if norm is not None else (None, None)
        if last and exit_norm is not None:
            if isinstance(exit_norm, RMSNorm) and exit_norm.groups == 1:
                return ops.add_rmsnorm(x, branch, weight, eps, exit_norm.weight, exit_norm.eps)
            ops.add_rmsnorm(x, branch, weight, eps, None, None)
            return exit_norm.forward(x)
        if self.runtime.exact:
            ops.add_rmsnorm(x, branch, weight, eps, None, None)
            return x
        return ops.add_rmsnorm(x, branch, weight, eps, None, None, rounded=True)

    def forward(self, x, h, ctx, exit_norm):
        if h is None:
            h = ops.rounded_rows(x, self.runtime.dtype)
        h = ops.settle(h)
        a = self.mixer.forward(h, ctx)
        h2 = self._step(x, a, self.norms["norm1"], exit_norm, self.feed_forward is None)
        if self.feed_forward is None:
            return x, h2
        m = self.feed_forward.forward(h2, ctx)
        return x, self._step(x, m, self.norms["norm2"], exit_norm, True)
