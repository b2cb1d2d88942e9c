"""Small Zafilix configurations for the tests, and folders with weights made so that every mechanism matters.

'mixed'   attention (grouped heads, value heads of their own size, a partial rotation with stretched frequencies, blocks of 24
          positions), two latent layers with windows of 21 and 40, a layer without a feed-forward, and three layers that run on
          earlier layers' tensors with caches of their own
'odd'     sizes in no step of 4 or 8 (width 50, heads of 10 and 6, a latent row of 20 + 6, feed-forwards of 30 and 14), one
          key/value head, a block no longer than a page, a window of one page and one token, no logit cap, no logit factor
'whole'   what a file may leave out is left out: no masks (every earlier key), no rotation in one layer, no stretch, as many
          key/value heads as query heads, an embedding factor of 1, latent layers first
'heads64' attention heads of 64 elements with values of the same size (the sizes that tensor-core attention kernels take),
          blocks of 48 and 80 positions, a latent row of 96 + 32 elements
"""
from __future__ import annotations

import copy
import json
import os

import torch
from safetensors.torch import save_file


def _att(heads, kv, dim, vdim=None, rot=None, scale=None, block=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim}
    if vdim is not None:
        m["vdim"] = vdim
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if len(rot) > 2:
            m["rot"]["scaling"] = {"factor": rot[2]}
    if scale is not None:
        m["scale"] = scale
    if block is not None:
        m["mask"] = {"size": block}
    return m


def _lat(heads, dim, rot_dim, vdim, rank, rot=None, scale=None, window=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if len(rot) > 2:
            m["rot"]["scaling"] = {"factor": rot[2]}
    if scale is not None:
        m["scale"] = scale
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _ff(n):
    return {"kind": "dense", "ff": n}


def _again(layers, j):
    layer = copy.deepcopy(layers[j])
    layer["weights_of"] = j
    return layer


_MIXED = [
    {"type": "attention", "mixer": _att(4, 2, 16, 24, (8, 500.0, 4.0), 0.3, 24), "mlp": _ff(48)},
    {"type": "latent_attention", "mixer": _lat(4, 16, 8, 12, 32, (8, 100.0), 0.21, 21), "mlp": _ff(40)},
    {"type": "latent_attention", "mixer": _lat(2, 24, 16, 16, 40, (16, 1000.0), 0.16, 40), "mlp": None},
    {"type": "attention", "mixer": _att(2, 1, 32, None, (32, 10000.0, 2.0), 0.2, 70), "mlp": _ff(56)},
]
MIXED = {
    "architecture": "Zafilix", "vocab": 200, "width": 64, "embedding": {"scale": 6.0}, "norm": {"eps": 1e-5},
    "logit_scale": 0.5, "logit_softcap": 9.0,
    "layers": _MIXED + [_again(_MIXED, 1), _again(_MIXED, 0), _again(_MIXED, 2)],
}

_ODD = [
    {"type": "latent_attention", "mixer": _lat(3, 10, 6, 6, 20, (6, 30.0), 0.3, 17), "mlp": _ff(30)},
    {"type": "attention", "mixer": _att(5, 1, 10, 6, (4, 30.0, 8.0), 0.35, 16), "mlp": _ff(14)},
]
ODD = {
    "architecture": "Zafilix", "vocab": 77, "width": 50, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-6},
    "layers": _ODD + [_again(_ODD, 1)],
}

WHOLE = {
    "architecture": "Zafilix", "vocab": 90, "width": 40, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
    "layers": [
        {"type": "latent_attention", "mixer": _lat(2, 8, 8, 8, 16, (8, 50.0)), "mlp": _ff(24)},
        {"type": "attention", "mixer": _att(3, 3, 16, None, (16, 100.0)), "mlp": _ff(32)},
        {"type": "attention", "mixer": _att(1, 1, 8), "mlp": None},
    ],
}

_HEADS64 = [
    {"type": "attention", "mixer": _att(6, 2, 64, None, (64, 10000.0, 4.0), 0.125, 48), "mlp": _ff(64)},
    {"type": "latent_attention", "mixer": _lat(4, 32, 32, 24, 96, (32, 10000.0), 0.12, 50), "mlp": _ff(64)},
    {"type": "attention", "mixer": _att(2, 2, 64, None, (32, 500.0), 0.125, 80), "mlp": None},
]
HEADS64 = {
    "architecture": "Zafilix", "vocab": 120, "width": 64, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6},
    "logit_scale": 0.2, "logit_softcap": 12.0,
    "layers": _HEADS64 + [_again(_HEADS64, 0)],
}

CONFIGS = {"mixed": MIXED, "odd": ODD, "whole": WHOLE, "heads64": HEADS64}
SEEDS = {"mixed": 31, "odd": 32, "whole": 33, "heads64": 34}


def write_folder(folder: str, name: str, dtype=torch.bfloat16) -> str:
    """config.json and model.safetensors.  Matrices N(0, 0.1); the gains of the norms behind the sublayers and of the last
    norm are stored around zero (the model adds one), the gains of the q, k and latent norms around one."""
    from wllm_b200.weights import random_tensors
    cfg = copy.deepcopy(CONFIGS[name])
    tensors = random_tensors(cfg, SEEDS[name], dtype=torch.float32, std=0.1, vector_std=0.3)
    for key, t in tensors.items():
        if key.endswith((".q.norm", ".k.norm", ".dkv.norm")):
            tensors[key] = 1.0 + t
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    save_file({k: v.to(dtype).contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder
