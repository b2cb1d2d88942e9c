"""Routed experts: a feed-forward in which every token runs a few of many small gated units.

spec options: num_experts, top, groups, groups_kept (the experts form `groups` equal groups of neighbours; a group's score
is its best expert's and only experts of the `groups_kept` best groups can be chosen; 1 and 1: no such limit), router
(checkpoint name of the router matrix [experts, hidden]), expert_prefix (expert j's tensors are <prefix><j>.gate / .up /
.down), intermediate_size, activation, limit, slope (the experts' gated unit, as 'gated_dense' takes them), scores ('softmax',
the default, over all experts; 'sigmoid': expert by expert, not normalised), gated (default True; False: an expert is
down(act(up x)) with tensors <prefix><j>.up / .down and activation 'relu_squared'), weight_on ('output', the default: the
chosen experts' outputs are multiplied by their scores; 'input': their inputs are, the output is the sum of expert(s x)), shared (None, or
the options of a 'gated_dense' unit that every token runs, plus gate_weight: the checkpoint name of one row [1, hidden]; the
unit's output is multiplied by sigmoid(row . x)).

Router logits, the softmax over all experts, the choice and the weights (the chosen experts' scores as they are) are
32-bit, against a 32-bit copy of the router matrix.  The tokens' (token, rank) pairs are sorted by expert on the device
and the experts run as two grouped products over the sorted rows (csrc/moe.cu; from `TC_FROM_PAIRS` pairs on, under
bfloat16, on the grouped form of the tensor-memory product, csrc/gemm_bf16_tc.cu); a token's output is the sum over its
ranks in rank order, so it does not depend on the batch beyond the rounding of the products.  Nothing comes back to the host, and every launch is sized
from the number of tokens and experts alone.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, ParamSpec, branch_pair, spec as make_spec


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts:
    graph_safe = True
    TC_FROM_PAIRS = 1024       # (token, expert) pairs from which the experts' products run on the tensor-memory kernel

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.E, self.top = int(spec.num_experts), int(spec.top)
        self.groups, self.groups_kept = int(spec.options.get("groups") or 1), int(spec.options.get("groups_kept") or 1)
        if self.E % self.groups or not 1 <= self.groups_kept <= self.groups or not 1 <= self.top <= self.groups_kept * (self.E // self.groups):
            raise ValueError(f"{self.E} experts in {self.groups} groups, {self.groups_kept} kept, top {self.top}: no such choice")
        self.inter, self.activation = int(spec.intermediate_size), spec.activation
        self.gated = bool(spec.options.get("gated", True))
        self.scores, self.weight_on = spec.options.get("scores") or "softmax", spec.options.get("weight_on") or "output"
        if self.scores not in ("softmax", "sigmoid") or self.weight_on not in ("output", "input"):
            raise ValueError(f"scores {self.scores!r} ('softmax', 'sigmoid'), weight_on {self.weight_on!r} ('output', 'input')")
        if self.activation != ("capped_swish" if self.gated else "relu_squared"):
            raise ValueError("the grouped expert products are built for gated experts with the activation capped_swish and for "
                             "experts without a gate with relu_squared")
        if self.weight_on == "input" and self.gated:
            raise ValueError("scores on the experts' inputs are built for experts without a gate")
        self.limit, self.slope = float(spec.options.get("limit") or 0.0), float(spec.options.get("slope") or 0.0)
        self.router_name, self.prefix = spec.router, spec.expert_prefix
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.shared = self.gate_name = None
        shared = spec.options.get("shared")
        if shared is not None:
            shared = dict(shared)
            self.gate_name = shared.pop("gate_weight")
            self.shared = FEED_FORWARDS.build(make_spec("gated_dense", **shared), hidden_size=hidden_size, model_dtype=model_dtype)
        self.w_router = self.w_gate = self.w_gu = self.w_down = None

    def parts(self):
        return [] if self.shared is None else [self.shared]

    def param_specs(self):
        H, I = self.hidden_size, self.inter
        out = [ParamSpec(self.router_name, (self.E, H))]
        for j in range(self.E):
            p = f"{self.prefix}{j}."
            out += ([ParamSpec(p + "gate", (I, H))] if self.gated else []) + [ParamSpec(p + "up", (I, H)), ParamSpec(p + "down", (H, I))]
        if self.shared is not None:
            out += self.shared.param_specs() + [ParamSpec(self.gate_name, (1, H))]
        return out

    def load(self, fetch):
        self.w_router = fetch(self.router_name).to(torch.float32).contiguous()
        names = [f"{self.prefix}{j}." for j in range(self.E)]
        if self.gated:
            self.w_gu = torch.stack([torch.cat([fetch(p + "gate"), fetch(p + "up")], dim=0) for p in names]).contiguous()
        else:
            self.w_gu = torch.stack([fetch(p + "up") for p in names]).contiguous()
        self.w_down = torch.stack([fetch(p + "down") for p in names]).contiguous()
        if self.shared is not None:
            self.shared.load(fetch)
            self.w_gate = fetch(self.gate_name).to(torch.float32).reshape(-1).contiguous()

    def __call__(self, x: torch.Tensor, ctx):
        n, top, H = x.shape[0], self.top, self.hidden_size
        pairs = n * top
        chosen = ctx.buffer("moe_chosen", (n, top), torch.int32)
        weights = ctx.buffer("moe_weights", (n, top), torch.float32)
        gate = ctx.buffer("moe_gate", (n,), torch.float32) if self.shared is not None else None
        ops.moe_route(x, self.w_router, self.w_gate, chosen, weights, gate, self.groups, self.groups_kept, scores=self.scores)
        unit = None if self.gated else self.activation
        on_input = weights.view(-1) if self.weight_on == "input" else None
        index = ctx.buffer("moe_index", (2 * self.E + 1 + 2 * pairs,), torch.int32)
        count, offset = index[:self.E], index[self.E:2 * self.E + 1]
        order, place = index[2 * self.E + 1:2 * self.E + 1 + pairs], index[2 * self.E + 1 + pairs:]
        act = ctx.buffer("moe_act", (pairs, self.inter), self.model_dtype)
        y = ctx.buffer("moe_y", (pairs, H), torch.float32)
        # Many rows (portions of prompts): the products run on the tensor-memory kernel over row tiles of one expert each, on
        # the tokens' rows copied into sorted order.  Few rows (decoding) are bound by streaming the experts' weights, which
        # the kernel on mma.sync does from rows gathered on the fly.
        if pairs >= self.TC_FROM_PAIRS and x.dtype == torch.bfloat16 and ops.tc_grouped_ok(x, self.w_gu) and self.inter % 8 == 0:
            tiles = ctx.buffer("moe_tiles", (1 + 3 * ops.moe_row_tiles(pairs, self.E),), torch.int32)
            ops.moe_plan(chosen, count, offset, order, place, tiles, ctx.buffer("moe_plan", (ops.MOE_PLAN_SEGMENTS * self.E,), torch.int32))
            # (scores on the inputs: the rows are multiplied while they are copied, rounded once)
            rows = ops.moe_gather(x, order, top, ctx.buffer("moe_rows", (pairs, H), self.model_dtype), row_weights=on_input)
            ops.gemm_bf16_tc_grouped(rows, self.w_gu, act, tiles, self.gated, self.limit, self.slope, unit=unit)
            ops.gemm_bf16_tc_grouped(act, self.w_down, y, tiles, False)
        else:
            ops.moe_plan(chosen, count, offset, order, place)
            # (scores on the inputs: the up product is linear, so the score multiplies its 32-bit sums in front of the activation)
            ops.moe_grouped(x, self.w_gu, act, offset, order, top, self.gated, self.limit, self.slope, unit=unit, row_weights=on_input)
            ops.moe_grouped(act, self.w_down, y, offset, order, top, False)
        shared = branch_pair(self.shared(x, ctx)) if self.shared is not None else None
        out = ctx.buffer("moe_out", (n, H), torch.float32)
        return ops.moe_combine(y, place, None if self.weight_on == "input" else weights, shared, gate, out)
