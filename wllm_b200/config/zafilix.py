"""Zafilix configuration, read from its own config.json keys.

    architecture     "Zafilix"
    vocab, width     sizes of the vocabulary and of the residual stream
    embedding.scale  factor on the token's embedding row (absent: 1)
    norm.eps         the eps of every root-mean-square norm of the model
    logit_scale      factor on the logits (absent: 1)
    logit_softcap    c: logits become c * tanh(logits / c), after the factor (absent: as they are)
    layers[i]        {"type": "attention" | "latent_attention", "mixer": {...}, "mlp": {"kind": "dense", "ff": n} or
                     null, "weights_of": j (optional)}

A layer with `weights_of: j` has no tensors of its own: it runs on layer j's (mixer, feed-forward, norms) with a cache
of its own; the rest of its entry must equal layer j's, and layer j must own its tensors.

Mixer `attention`: heads, kv_heads (default heads), dim, vdim (default dim), scale (default dim^-1/2),
rot {dims, base, scaling: {factor}} (absent: no rotation; no scaling: the frequencies as they are),
mask {size}: a position sees the earlier positions of its own block of `size` positions (absent: every earlier key).
Mixer `latent_attention`: heads, dim (elements of a head's query and key that do not turn), rot_dim (those that do),
vdim, kv_rank (size of the cached latent row), scale (default (dim + rot_dim)^-1/2), rot {dims, base, scaling} over
the rot_dim part, mask {size}: a position sees itself and the size - 1 positions before it (absent: every earlier key).
Whatever a config.json leaves out does not exist.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .base import ConfigError, ConfigReader

MIXER_TYPES = ("attention", "latent_attention")


def _sub(r: ConfigReader, raw, where: str):
    if not isinstance(raw, dict):
        r.complain(f"{where} must be an object")
        return None
    return ConfigReader(raw, where)


def _take(r: ConfigReader, sub: ConfigReader) -> None:
    r.problems.extend(f"{sub.where}: {p}" for p in sub.problems)
    sub.problems = []


def _rot(r: ConfigReader, raw: dict, limit, where: str):
    if raw.get("rot") is None:
        return None
    rot = _sub(r, raw["rot"], where + ".rot")
    if rot is None:
        return None
    out = {"dims": rot.integer("dims", minimum=0), "base": rot.number("base")}
    _take(r, rot)
    if out["dims"] is not None and limit and (out["dims"] % 2 or out["dims"] > limit):
        r.complain(f"{where}.rot.dims = {out['dims']}: even and at most {limit}")
    if raw["rot"].get("scaling") is not None:
        scaling = _sub(r, raw["rot"]["scaling"], where + ".rot.scaling")
        if scaling is not None:
            out["scaling"] = {"factor": scaling.number("factor")}
            _take(r, scaling)
    return out


def _mask(r: ConfigReader, raw: dict, where: str):
    if raw.get("mask") is None:
        return None
    mask = _sub(r, raw["mask"], where + ".mask")
    if mask is None:
        return None
    out = {"size": mask.integer("size")}
    _take(r, mask)
    return out


def _mixer(r: ConfigReader, kind: str, raw, where: str) -> dict:
    sub = _sub(r, raw, where)
    if sub is None:
        return {}
    heads, dim = sub.integer("heads"), sub.integer("dim")
    if kind == "attention":
        out = {"heads": heads, "kv_heads": sub.integer("kv_heads", default=heads), "dim": dim,
               "vdim": sub.integer("vdim", default=dim),
               "scale": sub.number("scale", default=(float(dim) ** -0.5 if dim else None))}
        turned = dim
        if heads and out["kv_heads"] and heads % out["kv_heads"]:
            r.complain(f"{where}: {heads} heads are no multiple of {out['kv_heads']} kv_heads")
    else:
        rot_dim = sub.integer("rot_dim", minimum=0)
        out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": sub.integer("vdim"), "kv_rank": sub.integer("kv_rank"),
               "scale": sub.number("scale", default=(float(dim + rot_dim) ** -0.5 if dim and rot_dim is not None else None))}
        turned = rot_dim
    _take(r, sub)
    rot, mask = _rot(r, raw, turned, where), _mask(r, raw, where)
    if rot is not None:
        out["rot"] = rot
    if mask is not None:
        out["mask"] = mask
    return out


def _layer(r: ConfigReader, i: int, layer, checked: list) -> dict:
    where = f"layers[{i}]"
    if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
        r.complain(f"{where}.type must be one of {', '.join(MIXER_TYPES)}")
        return {}
    out = {"type": layer["type"], "mixer": _mixer(r, layer["type"], layer.get("mixer"), where + ".mixer"), "mlp": None}
    mlp = layer.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
            r.complain(f"{where}.mlp.kind must be 'dense' (or mlp null)")
        else:
            sub = ConfigReader(mlp, where + ".mlp")
            out["mlp"] = {"kind": "dense", "ff": sub.integer("ff")}
            _take(r, sub)
    src = layer.get("weights_of")
    if src is not None:
        if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
            r.complain(f"{where}.weights_of = {src!r}: an earlier layer")
        elif checked[src]:
            if checked[src].get("weights_of") is not None:
                r.complain(f"{where}.weights_of = {src}: that layer has no tensors of its own")
            elif {k: v for k, v in checked[src].items() if k != "weights_of"} != out:
                r.complain(f"{where}: a layer that runs on layer {src}'s tensors must equal it in everything else")
            out["weights_of"] = src
    return out


@dataclass(frozen=True)
class ZafilixConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    logit_scale: float
    logit_softcap: float | None
    layers: tuple            # of checked layer dictionaries (see the module's text)

    architecture = "Zafilix"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "ZafilixConfig":
        r = ConfigReader(raw, where)
        vocab, width = r.integer("vocab"), r.integer("width")
        logit_scale = r.number("logit_scale", default=1.0)
        cap = r.number("logit_softcap", default=None)
        eps, scale = None, 1.0
        norm = _sub(r, raw.get("norm"), "norm")
        if norm is not None:
            eps = norm.number("eps")
            _take(r, norm)
        if raw.get("embedding") is not None:
            emb = _sub(r, raw["embedding"], "embedding")
            if emb is not None:
                scale = emb.number("scale", default=1.0)
                _take(r, emb)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            r.complain("'layers' must be a list with at least one layer")
            layers = []
        checked = []
        for i, layer in enumerate(layers):
            checked.append(_layer(r, i, layer, checked))
        r.finish()
        return cls(vocab=vocab, width=width, embedding_scale=scale, eps=eps, logit_scale=logit_scale, logit_softcap=cap,
                   layers=tuple(checked))

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs on."""
        src = self.layers[i].get("weights_of")
        return i if src is None else src

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "logit_scale": self.logit_scale,
             "layers": copy.deepcopy(list(self.layers))}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d


__all__ = ["ZafilixConfig", "ConfigError"]
