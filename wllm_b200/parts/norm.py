"""Norms over the model width with the residual add folded in.

'rmsnorm'    x / sqrt(mean(x^2) + eps) * gain.  spec options: weight (checkpoint name), eps, unit_offset (True: gain is
             1 + w, as Gemma stores it, src/wllm/models/gemma.py:42-51; False: gain is w).
'layernorm'  (x - mean(x)) / sqrt(mean((x - mean)^2) + eps) * w, a layer norm with a gain and no bias.
             spec options: weight, eps.
'identity'   nothing is normed: the residual (with the pending branch folded in) rounded to the model's element type, for
             blocks whose sublayers read the residual as it is.  No options, no tensors.
The statistics and the gain are applied in 32-bit on the 32-bit residual; the result is rounded once to the model's
element type.  `branch` norms a sublayer's output that has not joined the residual yet (blocks that norm behind
their sublayers as well as in front): its result stays 32-bit and becomes the residual's pending addend.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import NORMS, MeanOfNormed, NormedBranch, ParamSpec, Partials, Residual, branch_pair


@NORMS.register("rmsnorm")
class RMSNorm:
    graph_safe = True
    center = False

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.weight_name = spec.weight
        self.eps = float(spec.eps)
        self.offset = 1.0 if spec.options.get("unit_offset", False) else 0.0
        self.hidden_size = hidden_size
        self.model_dtype = model_dtype
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.weight_name, (self.hidden_size,), "vector")]

    def load(self, fetch):
        self.weight = fetch(self.weight_name)

    def __call__(self, residual: Residual, ctx) -> torch.Tensor:
        out = ctx.buffer("normed", (residual.stream.shape[0], self.hidden_size), self.model_dtype)
        self._run(residual, ctx, out, None)
        residual.pending = None
        return out

    def rows(self, residual: Residual, rows: torch.Tensor, ctx) -> torch.Tensor:
        out = torch.empty((rows.shape[0], self.hidden_size), dtype=self.model_dtype, device=rows.device)
        self._run(residual, ctx, out, rows)
        return out

    def _run(self, residual: Residual, ctx, out, rows) -> None:
        pending = residual.pending
        if isinstance(pending, NormedBranch) and self._fusable(pending):
            # the branch's own norm, the add and this norm in one kernel; two mixers' outputs are normed and averaged there too
            post, inner, more = pending.norm, pending.branch, {}
            if isinstance(inner, MeanOfNormed):
                more = dict(gain_a=inner.gain_a, b=branch_pair(inner.b), gain_b=inner.gain_b, inner_eps=inner.eps, factor=inner.factor)
                inner = inner.a
            ops.sandwich_norm(residual.stream, branch_pair(inner), out, post.weight, post.center, post.eps, self.weight,
                              self.offset, self.center, self.eps, rows=rows, post_offset=post.offset, **more)
            return
        delta, parts = residual.pending_args(ctx)
        extra = {"center": True} if self.center else {}
        if rows is not None:
            extra["rows"] = rows
        ops.rmsnorm(residual.stream, delta, self.weight, self.eps, self.offset, out, delta_splits=parts, **extra)

    def _fusable(self, pending: NormedBranch) -> bool:
        post = pending.norm
        if not isinstance(post, RMSNorm) or post.weight is None or self.hidden_size > 24 * 1024 or \
                (self.weight is not None and post.weight.dtype != self.weight.dtype):
            return False
        inner = pending.branch
        return not isinstance(inner, MeanOfNormed) or inner.gain_a.dtype == post.weight.dtype == inner.gain_b.dtype

    def branch(self, branch, ctx, name: str = "branch_normed") -> torch.Tensor:
        """The norm of a branch output (a tensor [n, hidden] or `Partials`), 32-bit."""
        pair = branch_pair(branch)
        out = ctx.buffer(name, (pair[0].shape[-2], self.hidden_size), torch.float32)
        return ops.branch_norm(pair, self.weight, out, self.eps, center=self.center, offset=self.offset)


@NORMS.register("layernorm")
class LayerNormNoBias(RMSNorm):
    center = True


@NORMS.register("identity")
class ResidualReader(RMSNorm):
    """No norm at all: what a sublayer reads when it reads the residual itself.  The pending branch is folded in (with
    its own norm, if it has one, in the same kernel) and the rows go out rounded to the model's element type."""

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.weight_name, self.weight = None, None
        self.eps, self.offset = 0.0, 0.0
        self.hidden_size, self.model_dtype = hidden_size, model_dtype

    def param_specs(self):
        return []

    def load(self, fetch):
        pass

    def branch(self, branch, ctx, name: str = "branch_normed"):
        raise TypeError("the identity norm reads the residual; it norms no branch")
