"""What a model is put together from: specs (data), parts (code), registries (names).

A *spec* says which part stands at a place and with which sizes and constants; it is
plain data made from the configuration, layer by layer.  A *part* is the code for one
kind of spec.  No part knows which model it is in: it gets its sizes, constants and
the checkpoint names of its tensors from its spec, and the step's batch from the
`StepContext`.  Five registries map a spec's `kind` to the class that runs it:

    NORMS          x (and a pending branch output) -> normed x
    POSITIONS      how a mixer encodes positions
    MIXERS         the part that mixes tokens (attention here); may need cache or state
    FEED_FORWARDS  the per-token part (dense, gated, experts)
    BLOCKS         how norms, mixer and feed-forward are arranged around the residual

Interfaces (duck-typed; see the built-in parts for examples):

    every part      __init__(spec, hidden_size, model_dtype), param_specs() -> [ParamSpec],
                    load(fetch) where fetch(name) returns the checkpoint tensor on the device
    norm            __call__(residual: Residual, ctx) -> tensor [n, hidden] in the model dtype
                    rows(residual, rows, ctx) -> the same at selected rows only
    position        an object the mixer of its kind understands (rotary: .inv_freq, .rotary_dim, and
                    optionally .pairing = 'half' | 'interleaved')
    mixer           cache_need() -> KVNeed | StateNeed | None, or a tuple of them (a mixer that reads pages
                    and keeps state of its own)
                    __call__(x, ctx, cache: CacheRef) -> tensor [n, hidden]
    feed-forward    __call__(x, ctx) -> tensor [n, hidden]
    block           __call__(residual, ctx, cache: CacheRef) -> None (updates the residual)
    embedding       __call__(token_ids, ctx) -> float32 tensor [n, hidden] (the residual stream)
    head            __init__(..., embedding) gets the model's embedding part (for a tied table);
                    __call__(hidden_rows, ctx) -> float32 logits [rows, vocab]

A part may declare `graph_safe = True`: everything it launches depends on device data and on the step's
size bounds alone (tokens, requests, table width, longest context rounded to the table's reach), never on
host copies of the batch's contents; its state slots it finds through the step's device arrays, and a request
that brings no token (length 0, a padded row of a captured step) leaves no trace.  Decode steps are replayed from
captured CUDA graphs only for models whose parts all say so; any other model runs every step eagerly, whatever
`cuda_graphs` asks for.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One checkpoint tensor a part reads.  kind: 'matrix' and 'table' are held in the
    model's element type; 'vector' (norm gains and the like) keeps a 32-bit storage type."""
    name: str
    shape: tuple
    kind: str = "matrix"


@dataclass(frozen=True)
class PartSpec:
    kind: str
    options: dict = field(default_factory=dict)

    def __getattr__(self, key: str) -> Any:
        try:
            return self.__dict__["options"][key]
        except KeyError:
            raise AttributeError(f"{self.kind} spec has no option '{key}'") from None


def spec(kind: str, **options) -> PartSpec:
    return PartSpec(kind, options)


@dataclass(frozen=True)
class KVNeed:
    """A mixer that reads keys and values from pages."""
    kv_heads: int
    head_dim: int
    window: int | None = None
    v_head_dim: int | None = None    # size of a value head when it differs from head_dim
    keep_first: int = 0              # with a window: the sequence's first keys that stay visible behind it
    blocks: bool = False             # `window` is the size of a block: a token reads the earlier keys of its own block of
                                     # that many positions (blocks counted from position 0) instead of the latest keys
    values_in_keys: bool = False     # a token's value is the first v_head_dim elements of its key's row: one pool holds both


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps per-request state of fixed size: name -> (shape, dtype)."""
    tensors: tuple   # of (name, shape, dtype)


@dataclass
class CacheRef:
    """Where a layer run finds its cache: pages of (group, layer), or state tensors by name.
    `writes` is false for a run that reads another run's cache."""
    group: int | None = None
    layer: int | None = None
    writes: bool = True
    state_names: dict | None = None   # mixer's own name -> name in the manager's state slots


class Partials:
    """A branch output still in parts: [parts, n, hidden] float32 partial sums (a split-K product), which the
    next norm adds in order while it folds them into the residual."""

    def __init__(self, tensor: torch.Tensor):
        self.tensor, self.parts = tensor, tensor.shape[0]


def branch_pair(branch) -> tuple:
    """(tensor, parts) of a branch output, as the norm kernels take it."""
    return (branch.tensor, branch.parts) if isinstance(branch, Partials) else (branch, 0)


class MeanOfNormed:
    """Two branch outputs whose sum is still to be taken: factor * (rms(a) * gain_a + rms(b) * gain_b), each normed over
    the model width.  The norm that meets it works it out inside its own kernel; `materialize` does it alone."""

    def __init__(self, a, gain_a, b, gain_b, eps: float, factor: float):
        self.a, self.gain_a, self.b, self.gain_b, self.eps, self.factor = a, gain_a, b, gain_b, eps, factor

    def materialize(self, ctx, name: str = "mean_of_normed") -> torch.Tensor:
        from ..kernels import ops
        pa, pb = branch_pair(self.a), branch_pair(self.b)
        out = ctx.buffer(name, tuple(pa[0].shape[-2:]), torch.float32)
        return ops.branch_norm(pa, self.gain_a, out, self.eps, center=False, factor=self.factor, b=pb, weight_b=self.gain_b)


class NormedBranch:
    """A branch output that is to pass a norm of its own before it joins the residual (a block that norms behind its
    sublayers): `branch` is a tensor, `Partials` or `MeanOfNormed`, `norm` the norm part.  The next norm of the
    residual does both in one kernel when it can; `materialize` runs the branch's norm alone."""

    def __init__(self, branch, norm):
        self.branch, self.norm = branch, norm

    def materialize(self, ctx, name: str = "branch_normed") -> torch.Tensor:
        inner = self.branch.materialize(ctx) if isinstance(self.branch, MeanOfNormed) else self.branch
        return self.norm.branch(inner, ctx, name)


def as_branch(product):
    """What ops.project returned, as a branch output: a tensor, or Partials."""
    tensor, parts = product
    return Partials(tensor) if parts else tensor


class Residual:
    """The residual stream in 32-bit, and the branch output not yet added to it (a tensor [n, hidden], or
    `Partials`).  The next norm folds `pending` in (one kernel), so no separate add is launched."""

    def __init__(self, stream: torch.Tensor):
        self.stream = stream
        self.pending = None

    def pending_args(self, ctx=None) -> tuple:
        """(delta tensor or None, number of parts) for the norm kernel."""
        if hasattr(self.pending, "materialize"):
            self.pending = self.pending.materialize(ctx)
        if isinstance(self.pending, Partials):
            return self.pending.tensor, self.pending.parts
        return self.pending, 0


class Registry(dict):
    def __init__(self, what: str):
        super().__init__()
        self.what = what

    def register(self, kind: str):
        def wrap(cls):
            self[kind] = cls
            return cls
        return wrap

    def build(self, part_spec: PartSpec, **kwargs):
        if part_spec.kind not in self:
            raise KeyError(f"no {self.what} of kind '{part_spec.kind}' is registered (known: {', '.join(sorted(self))})")
        return self[part_spec.kind](part_spec, **kwargs)


EMBEDDINGS = Registry("embedding")
HEADS = Registry("logits head")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block arrangement")
