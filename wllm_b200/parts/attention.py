"""Attention over the paged cache: fused q|k|v projection, rotary encoding and cache
write, attention, output projection.

spec options: num_heads, num_kv_heads, head_dim, position (a position spec),
window (None or a number of keys), q_proj/k_proj/v_proj/o_proj (checkpoint names).
Query head h reads key/value head h // (num_heads/num_kv_heads); scores are scaled
by head_dim^-0.5 (src/wllm/models/llama.py:74-79, 242).  The three projections are
stored as one matrix [(nq + 2 nkv) * hd, hidden], rows in the order q, k, v, so one
product replaces three (the reference runs three, src/wllm/models/llama.py:103-105).
Further options, all off by default: value_dim (size of a value head when it is not
head_dim; the output projection then reads num_heads * value_dim columns), scale (the
score factor in place of head_dim^-0.5), sink (checkpoint name of one number per query
head that joins the softmax denominator as e^sink, without key or value),
qk_unit_norm_eps (rotated q and k heads are divided by their root mean square,
y / sqrt(mean(y^2) + eps), before the scores), softcap (c: a score becomes c * tanh(score / c) after the scale),
keep_first (with a window: the first keys of a sequence stay visible behind it, at their true positions: key j
is seen from position i when j <= i and (i - j < window or j < keep_first)), reads_other_cache (the mixer has no key
and value projections, names no k_proj and v_proj, and must stand in a run that reads another run's cache; its queries,
mask, scale and cap are its own), mask ('window', the default: `window` counts the latest keys; 'blocks': `window` is
the size of a block, and position i sees key j <= i when both lie in the same block of that many positions, blocks
counted from position 0 of the sequence), row_norm ({"q": name, "k": name, "eps": e}: the token's whole query row, all
heads at once, is divided by its root mean square and multiplied by the gain of that name, the key row likewise, in
front of the rotary turn), gate_proj (checkpoint name of a matrix [num_heads * value_dim, hidden]: the heads' outputs are
multiplied by the sigmoid of that projection of the mixer's input before the output projection; the gate is computed by
the same product as q, k and v), bias ({"q": name, "k": name, "v": name}: a bias row per projection, added to the
finished sums in 32-bit; with row_norm), distance_slopes (one number per query head: the score of key j from position i
loses slope_h * (i - j), after the scale and the cap), value_mix ({"weight": name, "role": 'first' | 'later', "key":
label}: the layers that share a label blend their values with those of the layer whose role is 'first', for the same
token: v <- (1 - w) v + w v_first with w the scalar tensor `weight`, in 32-bit; the blended values are what is cached.  The
first layer leaves its values in a buffer of the step; its own `weight` tensor is read and not used).

A mixer may be one of several that read the same input (a block that runs two mixers side
by side): `input_weights()` lists the matrices that read the input, `mix(fused, parts,
col0, ...)` runs the mixer on its columns of a fused product that somebody else made.

One forward serves whole prompts, portions and decoded tokens alike: the step's keys
and values go into the pages first, then every token attends through its request's
block table.  Which kernels do that is decided here, from the step context's facts
about the batch: 32-bit (and head sizes the tensor-core kernels are not built for)
runs the one-warp-per-row kernel, by row or by row and chunk of keys; bfloat16 sends
requests with one token to the split-key decode kernel and the others to the tiled
prefill kernel, which find their requests by q_len on the device.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, POSITIONS, CacheRef, KVNeed, ParamSpec, as_branch


@MIXERS.register("attention")
class PagedAttention:
    graph_safe = True
    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.nq, self.nkv, self.hd = int(spec.num_heads), int(spec.num_kv_heads), int(spec.head_dim)
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads are no multiple of {self.nkv} key/value heads")
        self.window = spec.options.get("window")
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.borrows = bool(spec.options.get("reads_other_cache", False))
        self.names = {k: spec.options[k] for k in (("q_proj", "o_proj") if self.borrows else ("q_proj", "k_proj", "v_proj", "o_proj"))}
        cap = spec.options.get("softcap")
        self.softcap = 0.0 if cap is None else float(cap)
        self.keep_first = int(spec.options.get("keep_first") or 0) if self.window else 0
        if self.softcap < 0 or self.keep_first < 0:
            raise ValueError("softcap and keep_first must not be negative")
        mask = spec.options.get("mask") or "window"
        if mask not in ("window", "blocks"):
            raise ValueError(f"mask {mask!r}: 'window' or 'blocks'")
        self.blocks = mask == "blocks" and bool(self.window)
        if self.blocks and (self.keep_first or self.borrows):
            raise ValueError("a mask of blocks keeps no first keys and reads no other run's cache")
        self.row_norm = spec.options.get("row_norm")
        self.gate_name = spec.options.get("gate_proj")
        self.bias_names = spec.options.get("bias")
        slopes = spec.options.get("distance_slopes")
        self.slope_values = None if slopes is None else [float(v) for v in slopes]
        self.value_mix = spec.options.get("value_mix")
        if self.value_mix is not None and self.value_mix["role"] not in ("first", "later"):
            raise ValueError(f"value_mix role {self.value_mix['role']!r}: 'first' or 'later'")
        if (self.bias_names is not None or self.value_mix is not None) and (self.row_norm is None or self.borrows):
            raise ValueError("projection biases and blended values are built into the kernel that norms q and k as whole rows (row_norm)")
        if self.slope_values is not None and len(self.slope_values) != self.nq:
            raise ValueError(f"{len(self.slope_values)} distance slopes for {self.nq} query heads")
        if self.row_norm is not None and self.borrows:
            raise ValueError("row norms of q and k need the mixer's own key projection")
        self.position = POSITIONS.build(spec.position)
        self.vd = int(spec.options.get("value_dim") or self.hd)
        scale = spec.options.get("scale")
        self.scale = float(self.hd) ** -0.5 if scale is None else float(scale)
        # The kernels read heads in steps of 8 elements.  A head of another size is held with zeros behind it, in the
        # projections' rows (so that the products leave zeros there), in the pages and in the output projection's columns:
        # zeros add nothing to a score or to an output.  `hd_file` / `vd_file` are the checkpoint's sizes.
        self.hd_file, self.vd_file = self.hd, self.vd
        self.hd, self.vd = -(-self.hd // 8) * 8, -(-self.vd // 8) * 8
        if spec.options.get("qk_unit_norm_eps") is not None and self.hd != self.hd_file:
            raise ValueError(f"head size {self.hd_file}: heads that are divided by their root mean square come in steps of 8 elements")
        self.sink_name = spec.options.get("sink")
        self.unit_norm_eps = spec.options.get("qk_unit_norm_eps")
        # the tensor-core kernels take keys and values of one size; other cases run on the general kernels
        self.general = self.vd != self.hd
        # columns of the fused q|k|v row (q alone in a mixer that reads another's keys and values), the gate's behind them
        self.qkv_width = self.nq * self.hd if self.borrows else (self.nq + self.nkv) * self.hd + self.nkv * self.vd
        self.width = self.qkv_width + (self.nq * self.vd if self.gate_name is not None else 0)
        self.q_gain = self.k_gain = None
        self.tag = ""                    # set by a mixer that runs this one beside another: keeps their buffers apart
        self.wqkv = self.wo = self.sinks = self.bias = self.slopes = self.blend = None

    def cache_need(self):
        return KVNeed(self.nkv, self.hd, self.window, self.vd if self.vd != self.hd else None, self.keep_first, blocks=self.blocks)

    def param_specs(self):
        H, n = self.hidden_size, self.names
        out = [ParamSpec(n["q_proj"], (self.nq * self.hd_file, H)), ParamSpec(n["o_proj"], (H, self.nq * self.vd_file))]
        if not self.borrows:
            out[1:1] = [ParamSpec(n["k_proj"], (self.nkv * self.hd_file, H)), ParamSpec(n["v_proj"], (self.nkv * self.vd_file, H))]
        if self.sink_name is not None:
            out.append(ParamSpec(self.sink_name, (self.nq,), "vector"))
        if self.gate_name is not None:
            out.append(ParamSpec(self.gate_name, (self.nq * self.vd_file, H)))
        if self.row_norm is not None:
            out += [ParamSpec(self.row_norm["q"], (self.nq * self.hd_file,), "vector"),
                    ParamSpec(self.row_norm["k"], (self.nkv * self.hd_file,), "vector")]
        if self.bias_names is not None:
            out += [ParamSpec(self.bias_names["q"], (self.nq * self.hd_file,), "vector"),
                    ParamSpec(self.bias_names["k"], (self.nkv * self.hd_file,), "vector"),
                    ParamSpec(self.bias_names["v"], (self.nkv * self.vd_file,), "vector")]
        if self.value_mix is not None:
            out.append(ParamSpec(self.value_mix["weight"], (), "vector"))
        return out

    def load(self, fetch):
        n = self.names
        def heads_padded(w, heads, size, to):      # [heads * size, H] -> [heads * to, H] with zero rows behind every head
            if size == to:
                return w
            out = w.new_zeros((heads, to, w.shape[1]))
            out[:, :size] = w.view(heads, size, w.shape[1])
            return out.view(heads * to, w.shape[1])
        wq = heads_padded(fetch(n["q_proj"]), self.nq, self.hd_file, self.hd)
        if self.borrows:
            self.wqkv = wq.contiguous()
        else:
            self.wqkv = torch.cat([wq, heads_padded(fetch(n["k_proj"]), self.nkv, self.hd_file, self.hd),
                                   heads_padded(fetch(n["v_proj"]), self.nkv, self.vd_file, self.vd)], dim=0).contiguous()
        if self.gate_name is not None:
            self.wqkv = torch.cat([self.wqkv, heads_padded(fetch(self.gate_name), self.nq, self.vd_file, self.vd)], dim=0).contiguous()
        if self.row_norm is not None:
            gains = [heads_padded(fetch(self.row_norm[k])[:, None], heads, self.hd_file, self.hd)[:, 0].contiguous()
                     for k, heads in (("q", self.nq), ("k", self.nkv))]
            self.q_gain, self.k_gain = gains
        if self.bias_names is not None:
            rows = [heads_padded(fetch(self.bias_names[k]).to(torch.float32)[:, None], heads, size, to)[:, 0]
                    for k, heads, size, to in (("q", self.nq, self.hd_file, self.hd), ("k", self.nkv, self.hd_file, self.hd),
                                               ("v", self.nkv, self.vd_file, self.vd))]
            self.bias = torch.cat(rows).contiguous()
        if self.value_mix is not None:
            self.blend = fetch(self.value_mix["weight"]).to(torch.float32).reshape(1).contiguous()
        wo = fetch(n["o_proj"])
        self.wo = heads_padded(wo.t().contiguous(), self.nq, self.vd_file, self.vd).t().contiguous()
        if self.sink_name is not None:
            self.sinks = fetch(self.sink_name).to(torch.float32).contiguous()
        if self.slope_values is not None:
            self.slopes = torch.tensor(self.slope_values, dtype=torch.float64).to(torch.float32).to(self.wo.device)
        self.position.to(self.wo.device)

    def input_weights(self) -> list:
        return [self.wqkv]

    def __call__(self, x: torch.Tensor, ctx, cache: CacheRef):
        qkv, parts = ops.project(x, self.wqkv, lambda name, shape, dt: ctx.buffer(self.tag + "qkv_" + name, shape, dt))
        return self.mix(qkv, parts, 0, ctx, cache)

    def mix(self, fused: torch.Tensor, parts: int, col0: int, ctx, cache: CacheRef):
        """The mixer on columns col0 .. col0 + width of a fused product [n, W] (or partial sums [parts, n, W])."""
        if self.borrows and cache.writes:
            raise ValueError("an attention mixer without key and value projections must stand in a run that reads another run's cache")
        n = fused.shape[-2]
        qkv = fused if fused.shape[-1] == self.width else fused[..., col0:col0 + self.width]
        group = ctx.cache.groups[cache.group]
        k_pages, v_pages = group.keys(cache.layer), group.values(cache.layer)
        q = ctx.buffer(self.tag + "q_rotated", (n, self.nq * self.hd), self.model_dtype)
        extra = {}
        if self.vd != self.hd:
            extra["vd"] = self.vd
        if self.unit_norm_eps is not None:
            extra["unit_norm_eps"] = float(self.unit_norm_eps)
        slots = ctx.group_slots[cache.group] if cache.writes else None
        pairing = getattr(self.position, "pairing", "half")
        if self.row_norm is not None:
            if self.unit_norm_eps is not None:
                raise ValueError("q and k are normed either as whole rows or head by head, not both")
            ops.rope_row_norm_kv_write(qkv, q, ctx.positions, slots, self.position.inv_freq, k_pages, v_pages, self.nq, self.nkv,
                                       self.hd, self.position.rotary_dim, group.page_size, self.q_gain, self.k_gain,
                                       float(self.row_norm["eps"]), self.nq * self.hd_file, self.nkv * self.hd_file,
                                       in_splits=parts, pairing=pairing, vd=self.vd, bias=self.bias, **self._blend_args(n, ctx))
        else:
            ops.rope_kv_write(qkv[..., :self.qkv_width] if self.width != self.qkv_width else qkv, q, ctx.positions, slots,
                              self.position.inv_freq, k_pages, v_pages, self.nq, 0 if self.borrows else self.nkv, self.hd,
                              self.position.rotary_dim, group.page_size, in_splits=parts, pairing=pairing, **extra)
        attn = ctx.buffer(self.tag + "attn", (n, self.nq * self.vd), self.model_dtype)
        self.attend(q, attn, k_pages, v_pages, ctx, cache.group)
        if self.gate_name is not None:
            ops.sigmoid_gate(attn, qkv, parts, self.qkv_width)
        return as_branch(ops.project(attn, self.wo, lambda name, shape, dt: ctx.buffer(self.tag + "branch_" + name, shape, dt)))

    def _blend_args(self, n: int, ctx) -> dict:
        """The buffer of the step in which the first layer of a label leaves its values, and this layer's part in it."""
        if self.value_mix is None:
            return {}
        first = ctx.buffer("values_first_" + str(self.value_mix["key"]), (n, self.nkv * self.vd), torch.float32)
        return {"v_first": first, "blend": self.blend, "mix": self.value_mix["role"]}

    def attend(self, q, out, k_pages, v_pages, ctx, group: int) -> None:
        """Attention of every token of the step over its request's pages of cache group `group`."""
        nq, nkv, hd, scale = self.nq, self.nkv, self.hd, self.scale
        window = -self.window if self.blocks else (self.window or 0)     # the kernels take a block size as a negative window
        ps, table = ctx.cache.page_size, ctx.group_tables[group]
        if q.dtype != torch.bfloat16 or not ops.mma_head_dim_ok(hd) or self.general:
            # Three kernels with one result, bit for bit, so the choice is one of speed alone.  Portions of prompts:
            # 32 rows of a request share every tile of keys.  Few rows over long contexts (decoding): a warp per
            # (row, chunk of 64 keys).  Otherwise a warp per row.
            extra = {"vd": self.vd, "sinks": self.sinks} if (self.general or self.sinks is not None) else {}
            if self.slopes is not None:
                extra["slopes"] = self.slopes
            if self.softcap > 0 or self.keep_first > 0:
                extra.update(cap=self.softcap, keep=self.keep_first)
            if ctx.num_multi > 0 and hd <= 256 and self.vd <= 256:
                ops.paged_attention_simt_tiled(q, out, k_pages, v_pages, ctx.req_q_start, ctx.req_q_len, ctx.req_ctx_len,
                                               table, ctx.max_q_len, nq, nkv, hd, ps, window, scale, **extra)
                return
            rows, chunks = q.shape[0] * nq, ops.simt_chunks(ctx.max_ctx, window, self.keep_first)
            scratch = None
            if chunks > 1 and rows <= 4096 and rows * chunks <= 65536:
                scratch = ctx.buffer(self.tag + "attention_chunks", (rows * chunks * (self.vd + 2),), torch.float32)
            ops.paged_attention_simt(q, out, k_pages, v_pages, ctx.token_req, ctx.positions, table, nq, nkv, hd, ps,
                                     window, scale, scratch, chunks, **extra)
            return
        decode = ctx.num_single > 0 and nq // nkv <= 16
        extra = {"sinks": self.sinks} if self.sinks is not None else {}
        # the kernels that walk a list of key tiles (mma.sync) take a cap, kept first keys and a bias by distance
        listed = self.softcap > 0 or self.keep_first > 0 or self.slopes is not None
        if listed:
            extra.update(cap=self.softcap, keep=self.keep_first, slopes=self.slopes)
        if decode:
            R = ctx.n_requests
            # one CTA fits on an SM: every (request, kv head) is cut into parts so that the CTAs finish together
            # (planned for the context rounded up to 512 keys, so that a growing context seldom needs a new plan)
            split_keys, max_splits = ops.decode_split_plan(R * nkv, -(-ctx.max_ctx // 512) * 512, 32 if hd % 64 == 0 else 64)
            scratch = ctx.buffer(self.tag + "attention_splits", (ops.attention_mma_scratch_floats(R, nq, hd, max_splits),),
                                 torch.float32)
            ops.attention_mma_decode(q, out, k_pages, v_pages, ctx.req_q_start, ctx.req_q_len, ctx.req_ctx_len, table,
                                     nq, nkv, hd, ps, window, scale, split_keys, max_splits, scratch, **extra)
        if ctx.num_multi > 0 or not decode:
            # two CTAs share a tile only where both halves hold keys of every row: not with a list of tiles, and not with
            # blocks, where the rows behind a block's border see no key of the tile's first half
            split_above, halves = (0, None) if listed or self.blocks else self._shared_tiles(ctx, skip_single=decode)
            ops.attention_mma_prefill(q, out, k_pages, v_pages, ctx.req_q_start, ctx.req_q_len, ctx.req_ctx_len, table,
                                      ctx.max_q_len, nq, nkv, hd, ps, window, scale, skip_single=decode,
                                      split_above=split_above, halves=halves, **extra)

    def _shared_tiles(self, ctx, skip_single: bool):
        """Whether this step's prefill attention shares its heavy tiles between two CTAs (ops.prefill_share_plan),
        and the buffer for their partial results.  Worked out once a step and head layout (kept in the step's
        memo), not once a layer; head sizes that run on pairs of CTAs (steps of 128, more than one tile of rows)
        never share."""
        nq, nkv, hd = self.nq, self.nkv, self.hd
        key = ("attention_share", nq, nkv, hd, skip_single)
        if key not in ctx.memo:
            if hd % 128 == 0 and ctx.max_q_len * (nq // nkv) > 128:
                plan = 0
            else:
                plan = ops.prefill_share_plan(ctx.host["req_q_len"].tolist(), ctx.host["req_ctx_len"].tolist(), nq, nkv,
                                              hd, skip_single)
            ctx.memo[key] = plan
        split_above = ctx.memo[key]
        if split_above <= 0:
            return 0, None
        floats = ops.attention_prefill_halves_floats(ctx.n_requests, ctx.max_q_len, nq, nkv, hd)
        return split_above, ctx.buffer(self.tag + "attention_halves", (floats,), torch.float32)
