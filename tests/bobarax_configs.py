"""Tiny Bobarax configurations for the tests, and their random weights as a checkpoint would hold
them (matrices rounded to bfloat16, integer tables as they are). Their sizes are unlike one another
on purpose."""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch

from mlx_omnia_b200.registry import resolve_architecture


def _lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def _runs(heads, kv_heads, dim, vdim, size, scale, softcap):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "softcap": softcap, "mask": {"size": size}}}


def _window(heads, kv_heads, dim, vdim, dims, size, scale, base=300.0, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
             "rot": {"base": base, "dims": dims}, "mask": {"size": size}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": mixer}


def _dense(layer, ff):
    layer["mlp"] = {"kind": "dense", "ff": ff}
    return layer


def _moe(layer, ff, experts, top, limit):
    layer["mlp"] = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    return layer


def _bare(layer):
    layer["mlp"] = None
    return layer


CONFIGS = {
    # values wider and narrower than keys (the generic attention kernel in both precisions), two query
    # heads to a key head, a rotation over half of a head, windows and runs that are no multiple of
    # anything, two experts a token, a reader of another layer's cache, a layer without a feed-forward
    "K": {"architecture": "Bobarax", "vocab": 157, "width": 96, "residual_mult": 0.4, "logit_scale": 0.7,
          "norm": {"eps": 1e-5},
          "layers": [_dense(_lightning(3, 16, 24, (0.5, 0.9, 0.97)), 80),
                     _moe(_window(4, 2, 16, 8, 8, 7, 0.25), 24, 5, 2, 0.9),
                     _bare(_runs(4, 2, 16, 24, 11, 0.3, 5.0)),
                     _dense(_window(4, 2, 16, 8, 8, 5, 0.3, kv_from=1), 40),
                     _moe(_lightning(2, 8, 8, (0.8, 1.0)), 40, 3, 1, 2.0)]},
    # keys and values of one width (the tensor-core kernels in bfloat16), six query heads to a key
    # head, a whole-head rotation, runs first, a key width of 12 for the recurrence
    "L": {"architecture": "Bobarax", "vocab": 211, "width": 64, "residual_mult": 1.0, "logit_scale": 2.0,
          "norm": {"eps": 1e-6},
          "layers": [_moe(_runs(2, 2, 32, 32, 33, 0.18, 50.0), 32, 4, 3, 1.5),
                     _dense(_window(6, 1, 16, 16, 16, 9, 0.25), 48),
                     _dense(_lightning(5, 12, 20, (0.3, 0.6, 0.9, 0.99, 0.999)), 96),
                     _dense(_window(6, 1, 16, 16, 16, 20, 0.25, kv_from=1), 32),
                     _bare(_window(6, 1, 16, 16, 16, 9, 0.2, kv_from=1))]},
    # wider windows and runs for long prompts: edges of tiles (64), of decode chunks (128) and of pages;
    # heads of 64 over pages of 16 (the tcgen05 prefill kernel in bfloat16); a slow decay
    "M": {"architecture": "Bobarax", "vocab": 120, "width": 128, "residual_mult": 0.25, "logit_scale": 1.0,
          "norm": {"eps": 1e-5},
          "layers": [_dense(_window(4, 2, 64, 64, 32, 150, 0.125), 64),
                     _moe(_runs(4, 1, 24, 24, 130, 0.2, 30.0), 32, 6, 2, 1.0),
                     _dense(_lightning(4, 32, 16, (0.9, 0.99, 0.999, 0.9999)), 64),
                     _dense(_window(4, 2, 64, 64, 32, 70, 0.125, kv_from=0), 32)]},
    # nothing a multiple of eight: a width of 100, heads of 20 with values of 12, a window and a run of
    # a single token, every expert for every token, a rotation over four dims, a key width of 5
    "N": {"architecture": "Bobarax", "vocab": 101, "width": 100, "residual_mult": 0.6, "logit_scale": 1.5,
          "norm": {"eps": 1e-5},
          "layers": [_moe(_window(3, 3, 20, 12, 4, 1, 0.22), 20, 3, 3, 0.8),
                     _dense(_runs(5, 1, 36, 36, 1, 0.17, 2.0), 30),
                     _bare(_lightning(3, 5, 7, (0.7, 0.95, 0.5))),
                     _moe(_window(3, 3, 20, 12, 4, 6, 0.22, kv_from=0), 12, 2, 1, 0.5),
                     _dense(_runs(2, 2, 10, 14, 6, 0.3, 8.0), 20)]},
}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def tensors(name_or_raw, seed: int = 0) -> dict[str, torch.Tensor]:
    raw = config(name_or_raw) if isinstance(name_or_raw, str) else name_or_raw
    architecture = resolve_architecture(raw)
    drawn = architecture.random_tensors(architecture.parse(raw), seed)
    return {k: (t.to(torch.bfloat16).float() if t.is_floating_point() else t) for k, t in drawn.items()}


def prompt(length: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(700 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def write_folder(folder: Path, raw: dict, weights: dict[str, torch.Tensor]) -> None:
    """A model folder as the loader reads it: config.json, bfloat16 tensors and int32 tables."""
    from safetensors.torch import save_file

    folder.mkdir(parents=True, exist_ok=True)
    save_file({k: (t.to(torch.bfloat16) if t.is_floating_point() else t.to(torch.int32)).contiguous()
               for k, t in weights.items()}, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(raw))
