"""Small Gudarax configurations for the tests, and folders with weights made so that every mechanism matters.

'mixed'   a delta layer first, two attention layers that blend their values (windows of 21 and 40, grouped heads, values of
          their own size), a latent layer, a third attention layer with neither window nor blending and as many key/value
          heads as query heads, a second delta layer with as many query/key heads as value heads; dense and routed
          feed-forwards (2 of 6 experts), a layer without one; token inputs of 8 columns
'odd'     sizes in no step of 4 or 8 (width 50, heads of 10 and 6, latent rows of 20 and 14, a feed-forward of 14, 3 experts,
          token inputs of 5 columns, convolutions of 2 taps, a window of one page and one token)
'bare'    what a file may leave out is left out: no token input, no window, no blending, an embedding factor of 1;
          convolutions of one tap (no inputs kept), every expert chosen (top = experts), layers that begin with attention
'heads64' attention heads of 64 elements with values of the same size, a latent row of 96, delta heads of 64 by 64,
          blending between layers whose windows differ (40 and none)
"""
from __future__ import annotations

import copy
import json
import os

import torch
from safetensors.torch import save_file


def _att(heads, kv, dim, vdim=None, scale=None, window=None, v_mix=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim}
    if vdim is not None:
        m["vdim"] = vdim
    if scale is not None:
        m["scale"] = scale
    if window is not None:
        m["mask"] = {"size": window}
    if v_mix is not None:
        m["v_mix"] = v_mix
    return m


def _lat(heads, dim, vdim, rank, q_rank, scale=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank}
    if scale is not None:
        m["scale"] = scale
    return m


def _delta(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _ff(n):
    return {"kind": "dense", "ff": n}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


MIXED = {
    "architecture": "Gudarax", "vocab": 200, "width": 64, "max_positions": 400, "embedding": {"scale": 6.0}, "norm": {"eps": 1e-5},
    "token_side": {"dim": 8},
    "layers": [
        {"type": "delta", "mixer": _delta(4, 2, 16, 24, 4), "mlp": _moe(6, 2, 40)},
        {"type": "attention", "mixer": _att(4, 2, 16, 24, 0.3, 21, True), "mlp": _ff(48)},
        {"type": "latent_attention", "mixer": _lat(4, 16, 12, 32, 24, 0.21), "mlp": _moe(6, 2, 40)},
        {"type": "attention", "mixer": _att(4, 2, 32, 24, 0.2, 40, True), "mlp": None},
        {"type": "attention", "mixer": _att(2, 2, 16, None, None, None, False), "mlp": _ff(56)},
        {"type": "delta", "mixer": _delta(2, 2, 24, 16, 3), "mlp": _moe(4, 1, 32)},
    ],
}

ODD = {
    "architecture": "Gudarax", "vocab": 77, "width": 50, "max_positions": 300, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-6},
    "token_side": {"dim": 5},
    "layers": [
        {"type": "attention", "mixer": _att(5, 1, 10, 6, 0.35, 17, True), "mlp": _moe(3, 1, 14)},
        {"type": "delta", "mixer": _delta(3, 3, 10, 6, 2), "mlp": _ff(14)},
        {"type": "latent_attention", "mixer": _lat(3, 10, 6, 20, 14, 0.3), "mlp": _moe(3, 2, 14)},
        {"type": "attention", "mixer": _att(5, 1, 10, 6, 0.35, 16, True), "mlp": _ff(30)},
    ],
}

BARE = {
    "architecture": "Gudarax", "vocab": 90, "width": 40, "max_positions": 300, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _att(3, 3, 16), "mlp": _moe(2, 2, 24)},
        {"type": "delta", "mixer": _delta(2, 1, 8, 8, 1), "mlp": None},
        {"type": "latent_attention", "mixer": _lat(2, 8, 8, 16, 16), "mlp": _ff(24)},
    ],
}

HEADS64 = {
    "architecture": "Gudarax", "vocab": 120, "width": 64, "max_positions": 512, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6},
    "token_side": {"dim": 16},
    "layers": [
        {"type": "attention", "mixer": _att(6, 2, 64, None, 0.125, 40, True), "mlp": _ff(64)},
        {"type": "latent_attention", "mixer": _lat(4, 32, 24, 96, 64, 0.12), "mlp": _moe(4, 2, 64)},
        {"type": "delta", "mixer": _delta(2, 1, 64, 64, 4), "mlp": _ff(64)},
        {"type": "attention", "mixer": _att(6, 2, 64, None, 0.125, None, True), "mlp": _moe(4, 1, 64)},
    ],
}

CONFIGS = {"mixed": MIXED, "odd": ODD, "bare": BARE, "heads64": HEADS64}
SEEDS = {"mixed": 41, "odd": 42, "bare": 43, "heads64": 44}


def write_folder(folder: str, name: str, dtype=torch.bfloat16) -> str:
    """config.json and model.safetensors.  Matrices N(0, 0.1); the gains of all norms around one; the blending weights inside
    (0, 1); the decays' logarithms and biases such that the decays spread over (0, 1); the routers large enough for the scores
    to differ; the tables of token inputs of order one."""
    from wllm_b200.weights import random_tensors
    cfg = copy.deepcopy(CONFIGS[name])
    tensors = random_tensors(cfg, SEEDS[name], dtype=torch.float32, std=0.1, vector_std=0.3)
    g = torch.Generator().manual_seed(SEEDS[name] + 1000)
    for key, t in tensors.items():
        if key.endswith(("norm", "norm1", "norm2")):
            tensors[key] = 1.0 + t
        elif key.endswith(".vmix"):
            tensors[key] = torch.rand((), generator=g) * 0.6 + 0.2
        elif key.endswith((".q.b", ".k.b", ".v.b")):
            tensors[key] = t * 2.0
        elif key.endswith(".conv"):
            tensors[key] = t * 5.0
        elif key.endswith((".mix.a", ".mix.b", ".router")):
            tensors[key] = t * 4.0
        elif key.endswith(".A_log"):
            tensors[key] = torch.rand(t.shape, generator=g) * 2.0 - 1.0
        elif key == "side.embed":
            tensors[key] = t * 10.0
        elif key == "pos":
            tensors[key] = t * 3.0
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    save_file({k: v.to(dtype).contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder
