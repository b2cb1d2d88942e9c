"""Dense feed-forwards: gated, down(act(gate(x)) * up(x)), and plain, down(act(up(x))).

Kind 'gated_dense'.

spec options: intermediate_size, activation ('gelu_tanh' for Gemma's GeGLU,
src/wllm/models/gemma.py:54-62; 'silu'; 'relu'; 'capped_swish' with `limit` and `slope`: the unit
g = min(gate x, limit), u = clamp(up x, -limit, limit), down(g * sigmoid(slope g) * (u + 1))),
gate_proj/up_proj/down_proj (checkpoint names).  gate and up are stored as one matrix [2 I, hidden] (gate rows first).  Under
bfloat16 one tensor-memory GEMM computes both products and applies act(gate) * up in its
epilogue, in 32-bit on the accumulators; otherwise one product feeds the activation kernel.

Kind 'dense' (no gate).  spec options: intermediate_size, activation ('relu_squared': max(z, 0)^2), up_proj/down_proj
(checkpoint names).  Under bfloat16 the activation is the epilogue of the up product, on the 32-bit accumulators.

Kind 'token_gated_table': a per-token addend made from the token itself.  A table holds a row per token id; the part reads
`dim` columns of it from `first_column` on (several layers share one table, each with columns of its own) and computes
out_proj(act(gate_proj x) * row).  spec options: table (checkpoint name), vocab_size, table_width (columns of the whole
table), first_column, dim, activation ('gelu_tanh'), gate_proj [dim, hidden], out_proj [hidden, dim] (checkpoint names).
It reads the step's token ids from the step context.  Only the part's own columns of the table are kept on the device.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, ParamSpec, as_branch


@FEED_FORWARDS.register("gated_dense")
class GatedDense:
    graph_safe = True
    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.inter = int(spec.intermediate_size)
        self.activation = spec.activation
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r}: one of {', '.join(ops.ACTIVATIONS)}")
        self.limit = float(spec.options.get("limit") or 0.0)
        self.slope = float(spec.options.get("slope") or 0.0)
        if self.activation == "capped_swish" and not (self.limit > 0 and self.slope > 0):
            raise ValueError("activation capped_swish needs a positive limit and slope")
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.names = {k: spec.options[k] for k in ("gate_proj", "up_proj", "down_proj")}
        self.wgu = self.wd = None

    def param_specs(self):
        H, I, n = self.hidden_size, self.inter, self.names
        return [ParamSpec(n["gate_proj"], (I, H)), ParamSpec(n["up_proj"], (I, H)), ParamSpec(n["down_proj"], (H, I))]

    def load(self, fetch):
        n = self.names
        self.wgu = torch.cat([fetch(n["gate_proj"]), fetch(n["up_proj"])], dim=0).contiguous()
        self.wd = fetch(n["down_proj"]).contiguous()

    def __call__(self, x: torch.Tensor, ctx):
        n = x.shape[0]
        h = ops.gated_linear(x, self.wgu, self.activation, ctx.buffer("ffn_act", (n, self.inter), self.model_dtype),
                             lambda shape, dtype: ctx.buffer("gate_up", shape, dtype),
                             **({"limit": self.limit, "slope": self.slope} if self.activation == "capped_swish" else {}))
        return as_branch(ops.project(h, self.wd, lambda name, shape, dt: ctx.buffer("branch_" + name, shape, dt)))


@FEED_FORWARDS.register("dense")
class Dense:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.inter = int(spec.intermediate_size)
        self.activation = spec.activation
        if self.activation not in ops.UNIT_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r}: one of {', '.join(ops.UNIT_ACTIVATIONS)}")
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.names = {k: spec.options[k] for k in ("up_proj", "down_proj")}
        self.wu = self.wd = None

    def param_specs(self):
        H, I, n = self.hidden_size, self.inter, self.names
        return [ParamSpec(n["up_proj"], (I, H)), ParamSpec(n["down_proj"], (H, I))]

    def load(self, fetch):
        self.wu = fetch(self.names["up_proj"]).contiguous()
        self.wd = fetch(self.names["down_proj"]).contiguous()

    def __call__(self, x: torch.Tensor, ctx):
        n = x.shape[0]
        h = ops.unit_linear(x, self.wu, self.activation, ctx.buffer("ffn_act", (n, self.inter), self.model_dtype),
                            lambda shape, dtype: ctx.buffer("ffn_up", shape, dtype))
        return as_branch(ops.project(h, self.wd, lambda name, shape, dt: ctx.buffer("branch_" + name, shape, dt)))


@FEED_FORWARDS.register("token_gated_table")
class TokenGatedTable:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.vocab, self.table_width = int(spec.vocab_size), int(spec.table_width)
        self.first, self.dim = int(spec.first_column), int(spec.dim)
        if self.first < 0 or self.first + self.dim > self.table_width:
            raise ValueError(f"columns {self.first} .. {self.first + self.dim} lie outside a table of {self.table_width} columns")
        self.activation = spec.activation
        if self.activation not in ops.TOKEN_GATE_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r}: one of {', '.join(ops.TOKEN_GATE_ACTIVATIONS)}")
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.names = {k: spec.options[k] for k in ("table", "gate_proj", "out_proj")}
        self.table = self.w_gate = self.w_out = None

    def param_specs(self):
        H, n = self.hidden_size, self.names
        return [ParamSpec(n["table"], (self.vocab, self.table_width), "table"), ParamSpec(n["gate_proj"], (self.dim, H)),
                ParamSpec(n["out_proj"], (H, self.dim))]

    def load(self, fetch):
        self.table = fetch(self.names["table"])[:, self.first:self.first + self.dim].contiguous()
        self.w_gate = fetch(self.names["gate_proj"]).contiguous()
        self.w_out = fetch(self.names["out_proj"]).contiguous()

    def __call__(self, x: torch.Tensor, ctx):
        n = x.shape[0]
        z, parts = ops.project(x, self.w_gate, lambda name, shape, dt: ctx.buffer("token_gate_" + name, shape, dt))
        g = ops.token_gate(z, parts, ctx.token_ids, self.table, self.activation, ctx.buffer("token_gated", (n, self.dim), self.model_dtype))
        return as_branch(ops.project(g, self.w_out, lambda name, shape, dt: ctx.buffer("token_branch_" + name, shape, dt)))
