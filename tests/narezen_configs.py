"""Tiny Narezen configurations for the tests, and their random weights as a checkpoint would hold
them (matrices rounded to bfloat16). Their sizes are unlike one another on purpose."""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch

from mlx_omnia_b200.registry import resolve_architecture


def _pair(left, right, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale}}


def _pair_2(left, right, left_scale, right_scale):
    return {"type": "parallel_2", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                            "right_scale": right_scale}}


def _keys_attention(heads, kv_heads, dim, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}


def _rotated_attention(heads, kv_heads, dim, vdim, scale, dims, base):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"base": base, "dims": dims}}


def _channel_decay(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def _retention(heads, dim, vdim, decay, dims, base):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": dims}}


def _recurrent(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def _moe(layer, ff, experts, top, shared):
    layer["mlp"] = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        layer["mlp"]["shared"] = {"ff": shared}
    return layer


def _bare(layer):
    layer["mlp"] = None
    return layer


CONFIGS = {
    # the recurrent block first, two experts a token, a layer without a feed-forward, one without a
    # shared expert, a rotation over half a head (attention) and over all of it (retention), values
    # narrower and wider than keys, three query heads to a key head
    "P": {"architecture": "Narezen", "vocab": 157, "width": 96, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-5},
          "logit_softcap": 12.0,
          "layers": [_moe(_recurrent(48, 3, 3), 24, 5, 2, 40),
                     _moe(_pair_2(_rotated_attention(6, 2, 16, 24, 0.3, 8, 300.0),
                                  _retention(3, 16, 8, (0.6, 0.93, 1.0), 16, 70.0), 0.8, 1.3), 32, 4, 1, None),
                     _bare(_pair(_keys_attention(4, 2, 16, 0.6), _channel_decay(2, 8, 24, 3.0), 1.1, 0.7)),
                     _moe(_pair(_keys_attention(2, 1, 32, 0.4), _channel_decay(3, 16, 16, 9.0), 0.5, 1.4), 16, 3, 3, 24)]},
    # heads of 64 over pages of 16 (the tensor-core attention kernels in bfloat16), a key width of 64 for
    # the recurrences, slow decays, one block and one tap in the recurrent layer, no soft cap; every
    # expert for every token, so that no choice can fall the other way in bfloat16 and every row of
    # logits can be held to the tolerance
    "Q": {"architecture": "Narezen", "vocab": 211, "width": 128, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-6},
          "layers": [_moe(_pair(_keys_attention(4, 2, 64, 0.125), _channel_decay(2, 64, 32, 16.0), 1.2, 1.1), 32, 3, 3, 48),
                     _moe(_recurrent(64, 1, 1), 32, 1, 1, 32),
                     _moe(_pair_2(_rotated_attention(4, 1, 64, 64, 0.125, 32, 50000.0),
                                  _retention(2, 64, 64, (0.99, 0.9995), 32, 1e6), 1.2, 0.5), 32, 2, 2, None),
                     _bare(_recurrent(96, 4, 4))]},
    # nothing a multiple of eight: a width of 100, heads of 20 and 12, key widths of 5 and 12 for the
    # recurrences, values of 7 and 20, every expert for every token, five taps, a rotation over four dims
    "R": {"architecture": "Narezen", "vocab": 101, "width": 100, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
          "logit_softcap": 30.0,
          "layers": [_moe(_pair_2(_rotated_attention(3, 3, 20, 12, 0.22, 4, 40.0),
                                  _retention(3, 5, 7, (0.7, 0.95, 0.5), 4, 10.0), 1.0, 1.0), 20, 3, 3, 12),
                     _moe(_pair(_keys_attention(5, 1, 12, 0.5), _channel_decay(1, 12, 20, 1.0), 2.0, 0.3), 12, 2, 1, None),
                     _moe(_recurrent(30, 5, 5), 20, 2, 2, 20),
                     _bare(_pair_2(_rotated_attention(2, 2, 10, 14, 0.3, 10, 1000.0),
                                   _retention(2, 6, 3, (1.0, 0.25), 6, 500.0), 0.4, 2.5))]},
}

DECAY_RANKS = {"P": 5, "Q": 16, "R": 3}
"""Inner widths of the decay maps (only the tensors say them)."""


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def tensors(name_or_raw, seed: int = 0, rank: int | None = None) -> dict[str, torch.Tensor]:
    """Random weights under the checkpoint's names, rounded to bfloat16; the decay maps' inner width
    is `rank` (the named configuration's own by default)."""
    raw = config(name_or_raw) if isinstance(name_or_raw, str) else name_or_raw
    if rank is None:
        rank = DECAY_RANKS.get(name_or_raw, 4) if isinstance(name_or_raw, str) else 4
    architecture = resolve_architecture(raw)
    drawn = architecture.random_tensors(architecture.parse(raw), seed)
    g = torch.Generator().manual_seed(seed + 99)
    for name in [n for n in drawn if n.endswith(".a1")]:
        width, out = drawn[name].shape[1], drawn[name[:-1] + "2"].shape[0]
        drawn[name] = torch.randn(rank, width, generator=g) * width ** -0.5
        drawn[name[:-1] + "2"] = torch.randn(out, rank, generator=g) * 2.0 * rank ** -0.5
    return {k: t.to(torch.bfloat16).float() for k, t in drawn.items()}


def prompt(length: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(900 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def write_folder(folder: Path, raw: dict, weights: dict[str, torch.Tensor]) -> None:
    """A model folder as the loader reads it: config.json and bfloat16 tensors."""
    from safetensors.torch import save_file

    folder.mkdir(parents=True, exist_ok=True)
    save_file({k: t.to(torch.bfloat16).contiguous() for k, t in weights.items()}, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(raw))
