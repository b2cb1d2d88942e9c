"""Gudarax configuration, read from its own config.json keys.

    architecture     "Gudarax"
    vocab, width     sizes of the vocabulary and of the residual stream
    max_positions    rows of the learned position table
    embedding.scale  factor on the token's embedding row (absent: 1)
    norm.eps         the eps of every root-mean-square norm of the model
    token_side.dim   columns of the per-layer token table that one layer reads (absent: the layers have no token input)
    layers[i]        {"type": "attention" | "latent_attention" | "delta", "mixer": {...}, "mlp": {...} or null}

Mixer `attention`: heads, kv_heads (default heads), dim, vdim (default dim), scale (default dim^-1/2), mask {size}: a
position sees itself and the size - 1 positions before it (absent: every earlier key), v_mix (default false: the layer's
values are its own).
Mixer `latent_attention`: heads, dim, vdim, kv_rank (the cached latent row), q_rank (the queries' latent row), scale
(default dim^-1/2).
Mixer `delta`: heads, kv_heads (default heads), dim, vdim, conv (taps of the short convolution).
mlp: {"kind": "dense", "ff": n} or {"kind": "moe", "expert": {"ff": n}, "router": {"experts": E, "top": k}}.
Whatever a config.json leaves out does not exist.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .base import ConfigError, ConfigReader

MIXER_TYPES = ("attention", "latent_attention", "delta")


def _sub(r: ConfigReader, raw, where: str):
    if not isinstance(raw, dict):
        r.complain(f"{where} must be an object")
        return None
    return ConfigReader(raw, where)


def _take(r: ConfigReader, sub: ConfigReader) -> None:
    r.problems.extend(f"{sub.where}: {p}" for p in sub.problems)
    sub.problems = []


def _grouped(r: ConfigReader, sub: ConfigReader, where: str):
    heads = sub.integer("heads")
    kv = sub.integer("kv_heads", default=heads)
    if heads and kv and heads % kv:
        r.complain(f"{where}: {heads} heads are no multiple of {kv} kv_heads")
    return heads, kv


def _mixer(r: ConfigReader, kind: str, raw, where: str) -> dict:
    sub = _sub(r, raw, where)
    if sub is None:
        return {}
    if kind == "attention":
        heads, kv = _grouped(r, sub, where)
        dim = sub.integer("dim")
        out = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": sub.integer("vdim", default=dim),
               "scale": sub.number("scale", default=(float(dim) ** -0.5 if dim else None)),
               "v_mix": sub.boolean("v_mix", default=False)}
        if raw.get("mask") is not None:
            mask = _sub(r, raw["mask"], where + ".mask")
            if mask is not None:
                out["mask"] = {"size": mask.integer("size")}
                _take(r, mask)
    elif kind == "latent_attention":
        dim = sub.integer("dim")
        out = {"heads": sub.integer("heads"), "dim": dim, "vdim": sub.integer("vdim"), "kv_rank": sub.integer("kv_rank"),
               "q_rank": sub.integer("q_rank"), "scale": sub.number("scale", default=(float(dim) ** -0.5 if dim else None))}
    else:
        heads, kv = _grouped(r, sub, where)
        out = {"heads": heads, "kv_heads": kv, "dim": sub.integer("dim"), "vdim": sub.integer("vdim"),
               "conv": sub.integer("conv")}
    _take(r, sub)
    return out


def _mlp(r: ConfigReader, raw, where: str):
    if raw is None:
        return None
    if not isinstance(raw, dict) or raw.get("kind") not in ("dense", "moe"):
        r.complain(f"{where}.kind must be 'dense' or 'moe' (or mlp null)")
        return None
    if raw["kind"] == "dense":
        sub = ConfigReader(raw, where)
        out = {"kind": "dense", "ff": sub.integer("ff")}
        _take(r, sub)
        return out
    expert, router = _sub(r, raw.get("expert"), where + ".expert"), _sub(r, raw.get("router"), where + ".router")
    out = {"kind": "moe", "expert": {}, "router": {}}
    if expert is not None:
        out["expert"] = {"ff": expert.integer("ff")}
        _take(r, expert)
    if router is not None:
        out["router"] = {"experts": router.integer("experts"), "top": router.integer("top")}
        _take(r, router)
        e, top = out["router"]["experts"], out["router"]["top"]
        if e and top and top > e:
            r.complain(f"{where}.router: top {top} of {e} experts")
    return out


@dataclass(frozen=True)
class GudaraxConfig:
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    eps: float
    side_dim: int | None
    layers: tuple            # of checked layer dictionaries (see the module's text)

    architecture = "Gudarax"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "GudaraxConfig":
        r = ConfigReader(raw, where)
        vocab, width, max_positions = r.integer("vocab"), r.integer("width"), r.integer("max_positions")
        eps, scale, side = None, 1.0, None
        norm = _sub(r, raw.get("norm"), "norm")
        if norm is not None:
            eps = norm.number("eps")
            _take(r, norm)
        if raw.get("embedding") is not None:
            emb = _sub(r, raw["embedding"], "embedding")
            if emb is not None:
                scale = emb.number("scale", default=1.0)
                _take(r, emb)
        if raw.get("token_side") is not None:
            ts = _sub(r, raw["token_side"], "token_side")
            if ts is not None:
                side = ts.integer("dim")
                _take(r, ts)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            r.complain("'layers' must be a list with at least one layer")
            layers = []
        checked, mixed = [], None
        for i, layer in enumerate(layers):
            at = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                r.complain(f"{at}.type must be one of {', '.join(MIXER_TYPES)}")
                checked.append({})
                continue
            one = {"type": layer["type"], "mixer": _mixer(r, layer["type"], layer.get("mixer"), at + ".mixer"),
                   "mlp": _mlp(r, layer.get("mlp"), at + ".mlp")}
            m = one["mixer"]
            if one["type"] == "attention" and m.get("v_mix"):
                # the layers that mix values read the first such layer's: their value rows have one size
                if mixed is None:
                    mixed = (m.get("kv_heads"), m.get("vdim"))
                elif mixed != (m.get("kv_heads"), m.get("vdim")):
                    r.complain(f"{at}.mixer: value rows of {m.get('kv_heads')} x {m.get('vdim')} cannot be mixed with the first "
                               f"such layer's {mixed[0]} x {mixed[1]}")
            checked.append(one)
        r.finish()
        return cls(vocab=vocab, width=width, max_positions=max_positions, embedding_scale=scale, eps=eps, side_dim=side,
                   layers=tuple(checked))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.side_dim is not None:
            d["token_side"] = {"dim": self.side_dim}
        return d


__all__ = ["GudaraxConfig", "ConfigError"]
