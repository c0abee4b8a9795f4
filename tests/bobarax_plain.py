"""Bobarax, written out plainly: one function per mechanism, whole sequences, no cache, float64
unless told otherwise. It shares nothing with the package; the engine is compared with it.

Notation: a sequence is T tokens; D the model width; H query heads in G key/value groups;
dk the query/key size of a head, dv its value size; tensors are a dict by checkpoint name;
`p` is a tensor-name prefix such as "l3.mix.".
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float, w: torch.Tensor | None = None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times w."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def centred_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The block norms and the final norm: the stored weight sits around zero and is applied as 1 + w."""
    return rms(x, eps, 1.0 + w.to(x.dtype))


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: of the first `dims` dims, dim 2i turns with dim 2i + 1 by
    position * base^(-2i/dims); the other dims pass."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None, None] * freq
    c, s = torch.cos(angle), torch.sin(angle)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], dim=-1)


def sees_window(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j when 0 <= i - j < size."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def sees_chunk(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j <= i of its own run of `size` positions, runs counted from position 0."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def softmax_heads(q, k, v, see, scale: float, softcap: float | None) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv], `see` [T, T]: every head's softmax attention, the
    scores scaled and then, with `softcap` c, replaced by c tanh(score / c). -> [T, H * dv]"""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~see, -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * dv)


def whole_projection_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x [T, heads * d]: one root mean square over all of a token's heads at once, a plain weight of that size."""
    return rms(x, eps, w.to(x.dtype))


def window_keys_and_values(h, W, p: str, m: dict, eps: float):
    """Keys (normed over the whole projection, then rotated) and values of a rotating layer with
    projections of its own: [T, G, dk], [T, G, dv]."""
    T, G, dk, dv, dt = h.shape[0], m["kv_heads"], m["dim"], m["vdim"], h.dtype
    k = whole_projection_norm(h @ W[p + "k"].to(dt).T, W[p + "k.norm"], eps).view(T, G, dk)
    k = rotate_pairs(k, torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    return k, (h @ W[p + "v"].to(dt).T).view(T, G, dv)


def window_attention(h, W, p: str, m: dict, eps: float, kv) -> torch.Tensor:
    """The rotating mixer: sliding window, queries normed over the whole projection and rotated, the
    heads' outputs multiplied by sigmoid(g h) ahead of the output projection. `kv` are its own keys
    and values or those of the layer it reads."""
    T, H, dk, dt = h.shape[0], m["heads"], m["dim"], h.dtype
    q = whole_projection_norm(h @ W[p + "q"].to(dt).T, W[p + "q.norm"], eps).view(T, H, dk)
    q = rotate_pairs(q, torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    out = softmax_heads(q, kv[0], kv[1], sees_window(T, m["mask"]["size"]), m["scale"], None)
    out = out * torch.sigmoid(h @ W[p + "g"].to(dt).T)
    return out @ W[p + "o"].to(dt).T


def chunk_attention(h, W, p: str, m: dict, eps: float) -> torch.Tensor:
    """The mixer without positions: queries and keys normed over the whole projection, scores capped
    by a tanh, every query looking back to the start of its own run of positions and no further."""
    T, H, G, dk, dv, dt = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"], h.dtype
    q = whole_projection_norm(h @ W[p + "q"].to(dt).T, W[p + "q.norm"], eps).view(T, H, dk)
    k = whole_projection_norm(h @ W[p + "k"].to(dt).T, W[p + "k.norm"], eps).view(T, G, dk)
    v = (h @ W[p + "v"].to(dt).T).view(T, G, dv)
    out = softmax_heads(q, k, v, sees_chunk(T, m["mask"]["size"]), m["scale"], m.get("softcap"))
    return out @ W[p + "o"].to(dt).T


def decayed_state_heads(q, k, v, decay, S0=None):
    """Per head S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, token by token from S0 (zeros).
    q, k [T, H, dk], v [T, H, dv] -> (o [T, H, dv], the last S [H, dk, dv])."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=q.dtype) if S0 is None else S0.clone()
    d = torch.as_tensor(decay, dtype=q.dtype)[:, None, None]
    o = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = d * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def lightning_mixer(h, W, p: str, m: dict, eps: float) -> torch.Tensor:
    """Linear attention with one decay a head: q, k, v through SiLU, the decayed sum above, all heads'
    outputs RMS-normed together with a plain weight, gated by sigmoid(g h), projected out."""
    T, H, dk, dv, dt = h.shape[0], m["heads"], m["dim"], m["vdim"], h.dtype
    silu = torch.nn.functional.silu
    q = silu(h @ W[p + "q"].to(dt).T).view(T, H, dk)
    k = silu(h @ W[p + "k"].to(dt).T).view(T, H, dk)
    v = silu(h @ W[p + "v"].to(dt).T).view(T, H, dv)
    o, _ = decayed_state_heads(q, k, v, m["decay"])
    o = rms(o.reshape(T, H * dv), eps, W[p + "norm"].to(dt))
    return (o * torch.sigmoid(h @ W[p + "g"].to(dt).T)) @ W[p + "o"].to(dt).T


def relu_glu(h, W, p: str) -> torch.Tensor:
    """down(relu(gate h) * (up h))."""
    dt = h.dtype
    return (torch.relu(h @ W[p + "gate"].to(dt).T) * (h @ W[p + "up"].to(dt).T)) @ W[p + "down"].to(dt).T


def clamped_expert(h, W, p: str, limit: float) -> torch.Tensor:
    """g = min(gate h, limit), u = clamp(up h, -limit, limit); down(g sigmoid(1.702 g) (u + 1))."""
    dt = h.dtype
    g = torch.clamp(h @ W[p + "gate"].to(dt).T, max=limit)
    u = torch.clamp(h @ W[p + "up"].to(dt).T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].to(dt).T


def table_experts(h, tokens: list[int], W, p: str, mlp: dict) -> torch.Tensor:
    """Every token's experts are the row of its id in an integer table; each counts 1 / top."""
    top = mlp["router"]["top"]
    table = W[p + "table"]
    y = torch.zeros_like(h)
    for t, token in enumerate(tokens):
        for e in table[token].tolist():
            y[t] += clamped_expert(h[t: t + 1], W, f"{p}e{e}.", mlp["expert"]["limit"])[0] / top
    return y


def forward(tokens: list[int], W: dict, cfg: dict, dtype=torch.float64, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence. `layers_out`, when a list, receives the residual after every layer."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = W["embed"].to(dtype)[tokens]
    held: dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        h = centred_norm(x, W[p + "norm1"], eps)
        if kind == "lightning":
            a = lightning_mixer(h, W, p + "mix.", m, eps)
        elif kind == "attention":
            a = chunk_attention(h, W, p + "mix.", m, eps)
        elif kind == "attention_2":
            if m.get("kv_from") is None:
                held[i] = window_keys_and_values(h, W, p + "mix.", m, eps)
            a = window_attention(h, W, p + "mix.", m, eps, held[i if m.get("kv_from") is None else m["kv_from"]])
        else:
            raise ValueError(f"layer {i}: unknown type {kind!r}")
        x = x + mult * centred_norm(a, W[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = centred_norm(x, W[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = relu_glu(h, W, p + "mlp.")
            elif mlp["kind"] == "moe":
                y = table_experts(h, tokens, W, p + "mlp.", mlp)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward {mlp['kind']!r}")
            x = x + mult * centred_norm(y, W[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = centred_norm(x, W["final.norm"], eps)
    return (x @ W["embed"].to(dtype).T) * cfg.get("logit_scale", 1.0)
