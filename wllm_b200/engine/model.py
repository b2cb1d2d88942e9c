"""The model that every architecture becomes: parts built from a plan, run in the plan's order.

`ComposedModel` knows no architecture.  It builds the blocks of the plan from the
part registries, sorts the layer runs into cache groups by what their mixers need
(runs whose mixers need the same heads, head size and window share a group and a
block table), names the per-request state tensors that mixers declare, and runs
    embedding -> runs in order -> final norm at the wanted rows -> head.
"""
from __future__ import annotations

import torch

from ..cache import CacheGroupSpec, StateSpec
from ..parts import BLOCKS, EMBEDDINGS, HEADS, NORMS, CacheRef, KVNeed, ModelPlan, Residual, StateNeed


class ComposedModel:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype):
        self.plan, self.dtype = plan, dtype
        kw = dict(hidden_size=plan.hidden_size, model_dtype=dtype)
        self.embedding = EMBEDDINGS.build(plan.embedding, **kw)
        self.blocks = [BLOCKS.build(b, **kw) for b in plan.blocks]
        self.final_norm = NORMS.build(plan.final_norm, **kw)
        self.head = HEADS.build(plan.head, embedding=self.embedding, **kw)
        self.group_specs, self.state_specs, self.cache_refs = self._assign_caches()
        # captured decode steps replay the launches their parts chose at capture (see parts/base.py); the run that
        # warms a capture up is undone for per-request state by the runner
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in self.parts() + self.blocks)
        self.loaded = False

    def _assign_caches(self):
        keys, layers, states, refs = [], [], [], []
        # a run whose cache other runs read keeps what the widest of their masks sees: the longest window (or every key)
        # and the most kept first keys
        readers = {}
        for run in self.plan.runs:
            if run.cache_from is not None:
                need = self.blocks[run.block].cache_need()
                readers.setdefault(run.cache_from, []).extend(n for n in (need if isinstance(need, (tuple, list)) else (need,))
                                                              if isinstance(n, KVNeed))
        for i, run in enumerate(self.plan.runs):
            if run.cache_from is not None:
                src = refs[run.cache_from]
                refs.append(CacheRef(src.group, src.layer, False, src.state_names))
                continue
            need = self.blocks[run.block].cache_need()
            ref = CacheRef()
            for one in need if isinstance(need, (tuple, list)) else (need,):
                if isinstance(one, KVNeed):
                    if ref.group is not None:
                        raise TypeError(f"run {i}: a mixer reads the pages of one cache group")
                    vd = one.v_head_dim if one.v_head_dim and one.v_head_dim != one.head_dim else None
                    window, keep = one.window, one.keep_first if one.window is not None else 0
                    for other in readers.get(i, ()):
                        if (other.kv_heads, other.head_dim, other.v_head_dim or other.head_dim) != (one.kv_heads, one.head_dim, one.v_head_dim or one.head_dim):
                            raise TypeError(f"a run that reads the cache of run {i} has other key/value heads than it")
                        window = None if window is None or other.window is None else max(window, other.window)
                        keep = max(keep, other.keep_first)
                    if (one.blocks or one.values_in_keys) and readers.get(i):
                        raise TypeError(f"run {i}: a cache of blocks or of values held in the keys' rows is read by its own run alone")
                    key = (one.kv_heads, one.head_dim, window, vd, keep if window is not None else 0,
                           bool(one.blocks) and window is not None, bool(one.values_in_keys))
                    if key not in keys:
                        keys.append(key)
                        layers.append(0)
                    g = keys.index(key)
                    ref.group, ref.layer = g, layers[g]
                    layers[g] += 1
                elif isinstance(one, StateNeed):
                    ref.state_names = ref.state_names or {}
                    for name, shape, dt in one.tensors:
                        ref.state_names[name] = f"run{i}.{name}"
                        states.append(StateSpec(ref.state_names[name], tuple(shape), dt))
                elif one is not None:
                    raise TypeError(f"run {i}: cache_need() returned {one!r}; expected KVNeed, StateNeed, None or a tuple of them")
            refs.append(ref)
        groups = []
        for (kvh, hd, window, vd, keep, blocks, inside), n in zip(keys, layers):
            name = ("all" if window is None else f"{'blocks' if blocks else 'window'}{window}") + (f"+first{keep}" if keep else "") + \
                f"-{kvh}x{hd}" + (f"v{vd}" if vd else "") + ("-in-keys" if inside else "")
            groups.append(CacheGroupSpec(name, n, kvh, hd, window, vd, keep, blocks, inside))
        return groups, states, refs

    # -- weights -------------------------------------------------------------------
    def parts(self):
        out = [self.embedding]
        for b in self.blocks:
            out.extend(b.parts())
        out.extend([self.final_norm, self.head])
        return out

    def param_specs(self) -> list:
        seen, out = set(), []
        for part in self.parts():
            for ps in part.param_specs():
                if ps.name in seen:
                    continue
                seen.add(ps.name)
                out.append(ps)
        return out

    def load(self, fetch) -> None:
        for part in self.parts():
            part.load(fetch)
        self.loaded = True

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once (the tied table counts once)."""
        seen, total = set(), 0
        todo = list(self.parts())
        while todo:
            part = todo.pop()
            todo.extend(part.parts() if hasattr(part, "parts") else [])     # a mixer made of mixers
            for t in vars(part).values():
                if isinstance(t, torch.Tensor) and t.data_ptr() not in seen and t.dim() >= 1 and t.numel() > 1:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    # -- one step ------------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        residual = Residual(self.embedding(ctx.token_ids, ctx))
        for run, ref in zip(self.plan.runs, self.cache_refs):
            self.blocks[run.block](residual, ctx, ref)
        if ctx.want_rows.shape[0] == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=ctx.token_ids.device)
        hidden = self.final_norm.rows(residual, ctx.want_rows, ctx)
        return self.head(hidden, ctx)
