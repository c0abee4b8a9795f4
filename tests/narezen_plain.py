"""Narezen, written out plainly: one function per mechanism, whole sequences, no cache, float64
unless told otherwise. It shares nothing with the package; the engine is compared with it.

Notation: a sequence is T tokens; D the model width; H query heads in G key/value groups; dk the
query/key size of a head, dv its value size; tensors are a dict by checkpoint name; `p` is a
tensor-name prefix such as "l3.mix.left."; `m` is that part's entry of the configuration.
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float, w: torch.Tensor | None = None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times w."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.to(x.dtype)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: of the first `dims` dims, dim i turns with dim i + dims / 2 by the angle
    position * base^(-2i / dims); the other dims pass."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None, None] * freq
    c, s = torch.cos(angle), torch.sin(angle)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sink_softmax_heads(q, k, v, scale: float, sink: torch.Tensor) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]: causal softmax attention of every head whose
    denominator holds one more term exp(sink_h), which has no key and no value. -> [T, H * dv]"""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    see = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = ((q[:, head] @ k[:, g].T) * scale).masked_fill(~see, -math.inf)
        top = torch.maximum(s.max(-1).values, sink[head].to(q.dtype))
        e = torch.exp(s - top[:, None])
        out[:, head] = (e @ v[:, g]) / (e.sum(-1) + torch.exp(sink[head].to(q.dtype) - top))[:, None]
    return out.reshape(T, H * dv)


def keys_as_values_attention(h, W, p: str, m: dict, eps: float) -> torch.Tensor:
    """Softmax attention without positions and without a value projection: the values are the
    projected keys as they leave the product; queries and keys are then divided by their root mean
    square, head by head; one learned sink a head."""
    T, H, G, dk, dt = h.shape[0], m["heads"], m["kv_heads"], m["dim"], h.dtype
    q = (h @ W[p + "q"].to(dt).T).view(T, H, dk)
    k = (h @ W[p + "k"].to(dt).T).view(T, G, dk)
    a = sink_softmax_heads(rms(q, eps), rms(k, eps), k, m["scale"], W[p + "sink"])
    return a @ W[p + "o"].to(dt).T


def rotated_attention(h, W, p: str, m: dict) -> torch.Tensor:
    """Softmax attention with rotated queries and keys and a one in the denominator."""
    T, H, G, dk, dv, dt = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"], h.dtype
    pos = torch.arange(T)
    q = rotate_half((h @ W[p + "q"].to(dt).T).view(T, H, dk), pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half((h @ W[p + "k"].to(dt).T).view(T, G, dk), pos, m["rot"]["dims"], m["rot"]["base"])
    v = (h @ W[p + "v"].to(dt).T).view(T, G, dv)
    a = sink_softmax_heads(q, k, v, m["scale"], torch.zeros(H, dtype=dt))
    return a @ W[p + "o"].to(dt).T


def decayed_state_heads(q, k, v, decay, S0=None):
    """q, k [T, H, dk], v [T, H, dv], decay [T, H, dk] (a factor per token, head and key channel):
    S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token. -> o [T, H, dv], S"""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=q.dtype) if S0 is None else S0.clone()
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out, S


def gated_linear_attention(h, W, p: str, m: dict, eps: float) -> torch.Tensor:
    """Linear attention whose state decays by a factor per key channel that the token itself sets
    through a low-rank map: alpha = sigmoid(a2 (a1 h) + b)^(1 / tau)."""
    T, H, dk, dv, dt = h.shape[0], m["heads"], m["dim"], m["vdim"], h.dtype
    q = (h @ W[p + "q"].to(dt).T).view(T, H, dk) * dk ** -0.5
    k = (h @ W[p + "k"].to(dt).T).view(T, H, dk)
    v = (h @ W[p + "v"].to(dt).T).view(T, H, dv)
    z = (h @ W[p + "a1"].to(dt).T) @ W[p + "a2"].to(dt).T + W[p + "a2.b"].to(dt)
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).view(T, H, dk)
    o, _ = decayed_state_heads(q, k, v, alpha)
    o = rms(o, eps, W[p + "norm"]).reshape(T, H * dv)
    return (o * silu(h @ W[p + "g"].to(dt).T)) @ W[p + "o"].to(dt).T


def retention(h, W, p: str, m: dict, eps: float) -> torch.Tensor:
    """Linear attention with one constant decay per head, rotated queries and keys, the keys times
    dk^-1/2 after the rotation; every head's output divided by its root mean square."""
    T, H, dk, dv, dt = h.shape[0], m["heads"], m["dim"], m["vdim"], h.dtype
    pos = torch.arange(T)
    q = rotate_half((h @ W[p + "q"].to(dt).T).view(T, H, dk), pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half((h @ W[p + "k"].to(dt).T).view(T, H, dk), pos, m["rot"]["dims"], m["rot"]["base"]) * dk ** -0.5
    v = (h @ W[p + "v"].to(dt).T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=dt)[None, :, None].expand(T, H, dk)
    o, _ = decayed_state_heads(q, k, v, decay)
    o = rms(o, eps).reshape(T, H * dv)
    return (o * silu(h @ W[p + "g"].to(dt).T)) @ W[p + "o"].to(dt).T


def side_by_side(h, W, p: str, m: dict, eps: float, kind: str) -> torch.Tensor:
    """Two mixers that read the same input; their outputs are added with a constant each."""
    if kind == "parallel":
        left = keys_as_values_attention(h, W, p + "left.", m["left"], eps)
        right = gated_linear_attention(h, W, p + "right.", m["right"], eps)
    else:
        left = rotated_attention(h, W, p + "left.", m["left"])
        right = retention(h, W, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]: y_t = bias + sum_j taps[:, K - 1 - j] x_(t - j), zeros ahead of the start."""
    T, K = x.shape[0], taps.shape[1]
    y = bias.to(x.dtype).expand(T, -1).clone()
    for j in range(min(K, T)):
        y[j:] += x[: T - j] * taps[:, K - 1 - j].to(x.dtype)
    return y


def gated_recurrent_unit(h, W, p: str, m: dict) -> torch.Tensor:
    """A recurrent block with a real-gated linear recurrence: S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t
    per channel, with a_t = exp(-8 r_t softplus(lam)); r and i are sigmoids of block-diagonal maps of u."""
    T, C, B, dt = h.shape[0], m["width"], m["blocks"], h.dtype
    y = gelu_tanh(h @ W[p + "y"].to(dt).T + W[p + "y.b"].to(dt))
    u = causal_conv(h @ W[p + "x"].to(dt).T + W[p + "x.b"].to(dt), W[p + "conv"], W[p + "conv.b"])
    ub = u.view(T, B, C // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ra"].to(dt), ub) + W[p + "ra.b"].to(dt)).reshape(T, C)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ri"].to(dt), ub) + W[p + "ri.b"].to(dt)).reshape(T, C)
    log_a = -8.0 * r * torch.nn.functional.softplus(W[p + "lam"].to(dt))
    a = torch.exp(log_a)
    S = torch.zeros(C, dtype=dt)
    out = torch.zeros(T, C, dtype=dt)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ W[p + "o"].to(dt).T


def gated_expert(h, W, p: str) -> torch.Tensor:
    dt = h.dtype
    return (silu(h @ W[p + "gate"].to(dt).T) * (h @ W[p + "up"].to(dt).T)) @ W[p + "down"].to(dt).T


def routed_experts(h, W, p: str, mlp: dict, chosen_out: list | None = None) -> torch.Tensor:
    """Sigmoid scores of the router's outputs; the `top` largest choose a token's experts; a chosen
    expert is given the token times its score (not the other way round: its output is not weighed);
    an expert that every token uses is added."""
    dt = h.dtype
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.sigmoid(h @ W[p + "router"].to(dt).T)
    chosen = torch.topk(s, top, dim=-1).indices
    if chosen_out is not None:
        chosen_out.append(chosen)
    out = torch.zeros_like(h)
    for e in range(E):
        rows = (chosen == e).any(-1).nonzero().flatten()
        if len(rows):
            out[rows] += gated_expert(h[rows] * s[rows, e][:, None], W, p + f"e{e}.")
    if mlp.get("shared") is not None:
        out = out + gated_expert(h, W, p + "shared.")
    return out


def forward(tokens: list[int], W: dict, cfg: dict, dtype=torch.float64, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence."""
    eps = cfg["norm"]["eps"]
    x = W["embed"].to(dtype)[torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, eps, W[p + "norm1"])
        if layer["type"] in ("parallel", "parallel_2"):
            a = side_by_side(h, W, p + "mix.", layer["mixer"], eps, layer["type"])
        elif layer["type"] == "rglru":
            a = gated_recurrent_unit(h, W, p + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        x = x + rms(a, eps, W[p + "norm1b"])
        if layer.get("mlp") is not None:
            m = routed_experts(rms(x, eps, W[p + "norm2"]), W, p + "mlp.", layer["mlp"])
            x = x + rms(m, eps, W[p + "norm2b"])
        if layers_out is not None:
            layers_out.append(x.clone())
    z = rms(x, eps, W["final.norm"]) @ W["head"].to(dtype).T
    cap = cfg.get("logit_softcap")
    return z if cap is None else cap * torch.tanh(z / cap)
