"""Attention over cached latent rows: every head's key and value are linear maps of one small row per token.

spec options: num_heads, plain_dim (elements of a head's query and key that do not turn), rot_dim (those that do),
value_dim, kv_rank (size of the latent row), scale (the score factor), window (None or a number of keys: a position sees
itself and the window - 1 keys before it), eps (of the latent row's norm), position (a rotary spec over the rot_dim part),
q_proj [heads * (plain_dim + rot_dim), hidden], down_proj [kv_rank + rot_dim, hidden], latent_norm [kv_rank],
up_k [heads * plain_dim, kv_rank], up_v [heads * value_dim, kv_rank], o_proj [hidden, heads * value_dim] (checkpoint names).

Two more options.  query_latent ({"rank": r, "down": name [r, hidden], "norm": name [r], "up": name [heads * plain_dim, r]};
without a turning part): the queries are up(rms(down h) * gain) instead of q_proj h, with the eps of the latent row's norm.
gate_proj (name of a matrix [heads * value_dim, hidden]): the heads' outputs are multiplied by the sigmoid of that
projection of the mixer's input before the output projection.  Both ride on the one fused product of the mixer's input.

With h the mixer's input: q = q_proj h, head by head [plain | turning]; the down projection gives the latent row
c = rms(first kv_rank rows) * gain and, behind it, one turning key part t shared by all heads.  Head a's key is
[up_k_a c | turned t], its value up_v_a c, its score scale * (q_a . k_a), softmax over the visible keys.

What is cached per token is [c | turned t] and nothing else.  The maps are folded into the queries and the outputs,
    q_a . [up_k_a c | t] = [up_k_a^T q_a,plain | q_a,turned] . [c | t],      sum_j p_j up_v_a c_j = up_v_a (sum_j p_j c_j),
so attention runs over the cached rows themselves: one key/value head that every query head reads, keys of
kv_rank + rot_dim elements, values the rows' first kv_rank elements (the cache group holds one pool: `values_in_keys`).
One fused product makes q and the down projection; `ops.latent_prepare` norms, turns and writes the cache row and lays
the queries out; `ops.head_linear` applies up_k^T head by head, the paged attention kernels run with their window,
`ops.head_linear` applies up_v, and the output projection follows.  Whole prompts, portions and decoded tokens are one
case.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, POSITIONS, CacheRef, KVNeed, ParamSpec, as_branch


@MIXERS.register("latent_attention")
class LatentAttention:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.heads, self.dim, self.rot = int(spec.num_heads), int(spec.plain_dim), int(spec.rot_dim)
        self.vd, self.rank = int(spec.value_dim), int(spec.kv_rank)
        self.window = spec.options.get("window")
        self.scale, self.eps = float(spec.scale), float(spec.eps)
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.position = POSITIONS.build(spec.position)
        if self.position.head_dim != self.rot:
            raise ValueError(f"the rotary encoding covers {self.position.head_dim} elements, the turning part has {self.rot}")
        # a cached row is held in steps of 8 elements (16-byte loads), zeros behind the turned part
        self.row = -(-(self.rank + self.rot) // 8) * 8
        self.qlat = spec.options.get("query_latent")
        self.gate_name = spec.options.get("gate_proj")
        self.names = {k: spec.options[k] for k in ("down_proj", "latent_norm", "up_k", "up_v", "o_proj")}
        if self.qlat is None:
            self.names["q_proj"] = spec.options["q_proj"]
            self.q_rank = 0
        else:
            if self.rot:
                raise ValueError("queries through a latent row of their own have no turning part")
            self.q_rank = int(self.qlat["rank"])
        self.q_width = self.q_rank if self.q_rank else self.heads * (self.dim + self.rot)
        self.gate_col = self.q_width + self.rank + self.rot
        self.width = self.gate_col + (self.heads * self.vd if self.gate_name is not None else 0)    # columns of the fused product
        self.tag = ""
        self.w_in = self.w_uk_t = self.w_uv = self.wo = self.gain = self.q_gain = self.w_uq = None

    def cache_need(self):
        return KVNeed(1, self.row, self.window, self.rank, 0, values_in_keys=True)

    def param_specs(self):
        H, n = self.hidden_size, self.names
        if self.qlat is None:
            out = [ParamSpec(n["q_proj"], (self.q_width, H))]
        else:
            out = [ParamSpec(self.qlat["down"], (self.q_rank, H)), ParamSpec(self.qlat["norm"], (self.q_rank,), "vector"),
                   ParamSpec(self.qlat["up"], (self.heads * self.dim, self.q_rank))]
        if self.gate_name is not None:
            out.append(ParamSpec(self.gate_name, (self.heads * self.vd, H)))
        return out + [ParamSpec(n["down_proj"], (self.rank + self.rot, H)),
                      ParamSpec(n["latent_norm"], (self.rank,), "vector"), ParamSpec(n["up_k"], (self.heads * self.dim, self.rank)),
                      ParamSpec(n["up_v"], (self.heads * self.vd, self.rank)), ParamSpec(n["o_proj"], (H, self.heads * self.vd))]

    def load(self, fetch):
        n = self.names
        mats = [fetch(n["q_proj"] if self.qlat is None else self.qlat["down"]), fetch(n["down_proj"])]
        if self.gate_name is not None:
            mats.append(fetch(self.gate_name))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.gain = fetch(n["latent_norm"]).contiguous()
        if self.qlat is not None:
            self.q_gain = fetch(self.qlat["norm"]).to(self.gain.dtype).contiguous()
            self.w_uq = fetch(self.qlat["up"]).contiguous()
        # up_k head by head, transposed: [heads, kv_rank, plain_dim], so that the queries' map is x W^T like every product
        self.w_uk_t = fetch(n["up_k"]).view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = fetch(n["up_v"]).view(self.heads, self.vd, self.rank).contiguous()
        self.wo = fetch(n["o_proj"]).contiguous()
        self.position.to(self.wo.device)

    def input_weights(self) -> list:
        return [self.w_in]

    def __call__(self, x: torch.Tensor, ctx, cache: CacheRef):
        fused, parts = ops.project(x, self.w_in, lambda name, shape, dt: ctx.buffer(self.tag + "latent_in_" + name, shape, dt))
        return self.mix(fused, parts, 0, ctx, cache)

    def mix(self, fused: torch.Tensor, parts: int, col0: int, ctx, cache: CacheRef):
        if not cache.writes:
            raise ValueError("a latent attention mixer writes its own cache")
        n, H, R, row = fused.shape[-2], self.heads, self.rank, self.row
        cols = fused if fused.shape[-1] == self.width else fused[..., col0:col0 + self.width]
        group = ctx.cache.groups[cache.group]
        pages = group.keys(cache.layer)
        # a product that left one tensor in the model's type holds the queries' plain parts as the next product reads them
        in_place = parts == 0 and cols.dtype == self.model_dtype
        q_plain = None if in_place or self.q_rank else ctx.buffer(self.tag + "latent_q_plain", (n, H * self.dim), self.model_dtype)
        q_mapped = ctx.buffer(self.tag + "latent_q", (n, H * row), self.model_dtype)
        cq = ctx.buffer(self.tag + "latent_cq", (n, self.q_rank), self.model_dtype) if self.q_rank else None
        ops.latent_prepare(cols, parts, ctx.positions, ctx.group_slots[cache.group], self.position.inv_freq, self.gain, self.eps,
                           pages, group.page_size, q_plain, q_mapped, H, self.dim, self.rot, self.position.rotary_dim, R, row,
                           pairing=getattr(self.position, "pairing", "half"), q_rank=self.q_rank, q_gain=self.q_gain, cq_out=cq)
        if self.q_rank:
            # the queries from their normed latent row: one more product, then head by head as below
            plain = ops.linear(cq, self.w_uq, ctx.buffer(self.tag + "latent_q_up", (n, H * self.dim), self.model_dtype)).view(n, H, self.dim)
        else:
            plain = cols[:, :self.q_width].unflatten(1, (H, self.dim + self.rot))[:, :, :self.dim] if in_place else q_plain.view(n, H, self.dim)
        ops.head_linear(plain, self.w_uk_t, q_mapped.view(n, H, row)[:, :, :R])
        mixed = ctx.buffer(self.tag + "latent_mixed", (n, H * R), self.model_dtype)
        self.attend(q_mapped, mixed, pages, ctx, cache.group)
        heads_out = ctx.buffer(self.tag + "attn", (n, H * self.vd), self.model_dtype)
        ops.head_linear(mixed.view(n, H, R), self.w_uv, heads_out.view(n, H, self.vd))
        if self.gate_name is not None:
            ops.sigmoid_gate(heads_out, cols, parts, self.gate_col)
        return as_branch(ops.project(heads_out, self.wo, lambda name, shape, dt: ctx.buffer(self.tag + "branch_" + name, shape, dt)))

    def attend(self, q, out, pages, ctx, group: int) -> None:
        """Every token of the step over its request's cached rows: one key/value head for all query heads, the values
        inside the keys' rows.  bfloat16 steps run on the tensor cores (64 rows of a request share every tile of keys; a
        step of single tokens cuts their keys into splits).  The three kernels of the general family give one result, bit for bit
        (portions of prompts: 32 rows share every tile of keys; few rows over long contexts: a warp per row and chunk
        of keys)."""
        H, row, R, window = self.heads, self.row, self.rank, self.window or 0
        ps, table = ctx.cache.page_size, ctx.group_tables[group]
        if self.model_dtype == torch.bfloat16 and ops.latent_mma_ok(H, R, row, ps) and (ctx.num_multi > 0 or H <= 64):
            split_tiles, max_splits, scratch = 0, 1, None
            if ctx.num_multi == 0:          # single tokens alone: their keys in splits, so that few requests fill the SMs
                requests = ctx.req_q_len.shape[0]
                split_tiles, max_splits = ops.latent_split_plan(requests, H, ctx.max_ctx, window)
                if split_tiles > 0:
                    scratch = ctx.buffer(self.tag + "latent_splits", (ops.latent_mma_scratch_floats(requests, H, R, max_splits),),
                                         torch.float32)
            ops.latent_attention_mma(q, out, pages, ctx.req_q_start, ctx.req_q_len, ctx.req_ctx_len, table, ctx.max_q_len,
                                     H, R, row, ps, window, self.scale, split_tiles=split_tiles, max_splits=max_splits,
                                     scratch=scratch)
            return
        if ctx.num_multi > 0 and row <= 256 and R % 8 == 0:
            ops.paged_attention_simt_tiled(q, out, pages, pages, ctx.req_q_start, ctx.req_q_len, ctx.req_ctx_len, table,
                                           ctx.max_q_len, H, 1, row, ps, window, self.scale, vd=R, values_in_keys=True)
            return
        rows, chunks = q.shape[0] * H, ops.simt_chunks(ctx.max_ctx, window)
        scratch = None
        if chunks > 1 and rows <= 4096 and rows * chunks <= 65536:
            scratch = ctx.buffer(self.tag + "attention_chunks", (rows * chunks * (R + 2),), torch.float32)
        ops.paged_attention_simt(q, out, pages, pages, ctx.token_req, ctx.positions, table, H, 1, row, ps, window, self.scale,
                                 scratch, chunks, vd=R, values_in_keys=True)
