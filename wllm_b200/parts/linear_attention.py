"""Linear attention with a decayed matrix state, and two mixers side by side.

'linear_attention': per head a state S [dim, vdim] that lives in 32-bit in the request's state slot,

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,    o_t = S_t^T q_t,

no softmax and no denominator.  Each head's o is divided by its root mean square over vdim (times a gain shared by
the heads, if the spec names one), the heads are multiplied by silu(g) and projected.  The decay is data:
    decay = {"kind": "per_head", "values": [a_0, ..]}         one constant per head (retention)
    decay = {"kind": "low_rank", "down": name, "up": name, "bias": name, "tau": t}
                                                              per key channel and token, sigmoid(up(down x) + bias)^(1/t)
                                                              (gated linear attention)
spec options: num_heads, key_dim, value_dim, eps, q_scale, k_scale (applied after the rotation), position (a rotary
spec, or None), decay, head_norm_weight (checkpoint name or None), q_proj/k_proj/v_proj/g_proj/o_proj (names).
All projections that read the mixer's input are one matrix, rows in the order q, k, v, g, down: one product.
What enters the recurrence is 32-bit (csrc/linear_attention.cu): the rotation, the scales, the decay and the state;
the projections run in the model's element type.

'parallel_mean': two mixers read the same input; each output is root-mean-square normed over the model width with a
gain of its own, and the result is half their sum.  One product serves both (`input_weights` / `mix`).
spec options: left, right (mixer specs), left_out, right_out (names of the gains), eps.
'delta_rule': the gated delta rule.  Per head a state S [dim, vdim] in the request's state slot, 32-bit; every token first
decays it, then corrects it towards its value along its key, then reads it with its query:

    S <- g_t S;    u_t = beta_t (v_t - S^T k_t);    S <- S + k_t u_t^T;    o_t = S^T q_t

q, k (num_kv_heads heads of key_dim; value head h reads q/k head h // (num_heads / num_kv_heads)) and v (num_heads heads of
value_dim) are each filtered along the sequence, channel by channel, by `conv_taps` taps that look back only (the last tap weighs
the token itself, inputs in front of the sequence count as zero; the newest taps - 1 inputs are kept as state) and pass SiLU; q and k heads are divided by sqrt(sum(x^2) +
unit_norm_eps), q is also multiplied by q_scale; beta_t = sigmoid(beta_proj x) and g_t = exp(-exp(decay_log) softplus(decay_proj x +
decay_bias)), one of each per head.  Each head's o is divided by its root mean square over value_dim (eps), times the gain
head_norm_weight shared by the heads, times silu(g_proj x); then o_proj.
spec options: num_heads, num_kv_heads, key_dim, value_dim, conv_taps, eps, unit_norm_eps, q_scale, q_proj/k_proj/v_proj/g_proj/
o_proj, q_conv/k_conv/v_conv [channels, taps], beta_proj, decay_proj [heads, hidden], decay_log, decay_bias [heads],
head_norm_weight [value_dim] (checkpoint names).  One product makes q | k | v | g | beta | decay; what enters the
recurrence is 32-bit (csrc/delta_rule.cu).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, POSITIONS, CacheRef, KVNeed, MeanOfNormed, ParamSpec, StateNeed, as_branch


@MIXERS.register("linear_attention")
class LinearAttention:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.heads, self.dim, self.vdim = int(spec.num_heads), int(spec.key_dim), int(spec.value_dim)
        if self.dim > 256:
            raise ValueError(f"key_dim {self.dim}: the recurrence kernel holds up to 256 key channels a head")
        self.eps = float(spec.eps)
        self.q_scale, self.k_scale = float(spec.options.get("q_scale", 1.0)), float(spec.options.get("k_scale", 1.0))
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.names = {k: spec.options[k] for k in ("q_proj", "k_proj", "v_proj", "g_proj", "o_proj")}
        self.position = POSITIONS.build(spec.position) if spec.options.get("position") is not None else None
        decay = dict(spec.decay)
        self.decay_kind = decay["kind"]
        if self.decay_kind == "per_head":
            if len(decay["values"]) != self.heads:
                raise ValueError(f"{len(decay['values'])} decays for {self.heads} heads")
            self.decay_values = [float(a) for a in decay["values"]]
        elif self.decay_kind == "low_rank":
            self.tau = float(decay["tau"])
            self.names.update(down=decay["down"], up=decay["up"], bias=decay["bias"])
            self.rank = None          # taken from the checkpoint's shapes when the spec does not say
            if "rank" in decay:
                self.rank = int(decay["rank"])
        else:
            raise ValueError(f"decay of kind {self.decay_kind!r}: per_head or low_rank")
        self.norm_name = spec.options.get("head_norm_weight")
        self.tag = ""
        self.w_in = self.wo = self.w_up = self.b_up = self.norm_weight = self.head_decay = None
        HD, HV = self.heads * self.dim, self.heads * self.vdim
        self.off_k, self.off_v, self.off_g, self.off_low = HD, 2 * HD, 2 * HD + HV, 2 * HD + 2 * HV

    def cache_need(self):
        return StateNeed((("state", (self.heads, self.dim, self.vdim), torch.float32),))

    def param_specs(self):
        H, n, HD, HV = self.hidden_size, self.names, self.heads * self.dim, self.heads * self.vdim
        out = [ParamSpec(n["q_proj"], (HD, H)), ParamSpec(n["k_proj"], (HD, H)), ParamSpec(n["v_proj"], (HV, H)),
               ParamSpec(n["g_proj"], (HV, H)), ParamSpec(n["o_proj"], (H, HV))]
        if self.decay_kind == "low_rank":
            out += [ParamSpec(n["down"], (self.rank, H)), ParamSpec(n["up"], (HD, self.rank)),
                    ParamSpec(n["bias"], (HD,), "vector")]
        if self.norm_name is not None:
            out.append(ParamSpec(self.norm_name, (self.vdim,), "vector"))
        return out

    def load(self, fetch):
        n = self.names
        mats = [fetch(n[k]) for k in ("q_proj", "k_proj", "v_proj", "g_proj")]
        if self.decay_kind == "low_rank":
            mats.append(fetch(n["down"]))
            self.w_up = fetch(n["up"]).contiguous()
            if mats[-1].shape[0] != self.w_up.shape[1]:
                raise ValueError(f"{n['down']} has {mats[-1].shape[0]} rows, {n['up']} reads {self.w_up.shape[1]}")
            self.rank = int(self.w_up.shape[1])
            self.b_up = fetch(n["bias"]).to(self.w_up.dtype).contiguous()
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.wo = fetch(n["o_proj"]).contiguous()
        if self.norm_name is not None:
            self.norm_weight = fetch(self.norm_name).contiguous()
        if self.decay_kind == "per_head":
            self.head_decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.wo.device)
        if self.position is not None:
            self.position.to(self.wo.device)

    def input_weights(self) -> list:
        return [self.w_in]

    @property
    def width(self) -> int:
        return self.off_low + (self.rank if self.decay_kind == "low_rank" else 0)

    def __call__(self, x: torch.Tensor, ctx, cache: CacheRef):
        fused, parts = ops.project(x, self.w_in, lambda name, shape, dt: ctx.buffer(self.tag + "la_in_" + name, shape, dt))
        return self.mix(fused, parts, 0, ctx, cache)

    def mix(self, fused: torch.Tensor, parts: int, col0: int, ctx, cache: CacheRef):
        """The mixer on the columns from col0 of a fused product [n, W] (or partial sums [parts, n, W])."""
        n, H, D, V, f32 = fused.shape[-2], self.heads, self.dim, self.vdim, torch.float32
        q = ctx.buffer(self.tag + "la_q", (n, H * D), f32)
        k = ctx.buffer(self.tag + "la_k", (n, H * D), f32)
        v = ctx.buffer(self.tag + "la_v", (n, H * V), f32)
        low = self.decay_kind == "low_rank"
        decay = ctx.buffer(self.tag + "la_decay", (n, H * D), f32) if low else None
        rot = self.position.rotary_dim if self.position is not None else 0
        ops.linattn_prepare(fused, parts, col0, col0 + self.off_k, col0 + self.off_v, H, D, V, ctx.positions, q, k, v,
                            q_scale=self.q_scale, k_scale=self.k_scale,
                            inv_freq=self.position.inv_freq if rot else None, rot_dim=rot,
                            low_off=col0 + self.off_low if low else -1, w2=self.w_up, b2=self.b_up,
                            tau=self.tau if low else 1.0, decay=decay)
        o = ctx.buffer(self.tag + "la_o", (n, H * V), f32)
        # long portions are cut into segments that run side by side; the plan is a function of the step's shape alone
        seg_len, max_seg = ops.linattn_segment_plan(ctx.max_q_len, ctx.num_multi, H, V)
        seg_state = seg_decay = None
        if max_seg > 1:
            R = ctx.n_requests
            seg_state = ctx.buffer(self.tag + "la_seg_state", (R * max_seg * H * D * V,), f32)
            seg_decay = ctx.buffer(self.tag + "la_seg_decay", (R * max_seg * H * D,), f32)
        ops.linattn_scan(q, k, v, decay, self.head_decay, ctx.state(cache.state_names["state"]), o, ctx.req_q_start,
                         ctx.req_q_len, ctx.req_slot, H, D, V, seg_len, max_seg, seg_state, seg_decay)
        gated = ctx.buffer(self.tag + "la_gated", (n, H * V), self.model_dtype)
        ops.head_gate_norm(o, fused, parts, col0 + self.off_g, self.norm_weight, self.eps, gated, H, V)
        return as_branch(ops.project(gated, self.wo, lambda name, shape, dt: ctx.buffer(self.tag + "la_out_" + name, shape, dt)))


@MIXERS.register("parallel_mean")
class ParallelMean:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        kw = dict(hidden_size=hidden_size, model_dtype=model_dtype)
        self.left, self.right = MIXERS.build(spec.left, **kw), MIXERS.build(spec.right, **kw)
        for side, m in (("left", self.left), ("right", self.right)):
            if not hasattr(m, "mix") or not hasattr(m, "input_weights"):
                raise TypeError(f"the {side} mixer ({type(m).__name__}) cannot share a fused input product")
            m.tag = side + "_" + getattr(m, "tag", "")
        self.eps = float(spec.eps)
        self.names = {"left": spec.left_out, "right": spec.right_out}
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.w_in = self.gain_left = self.gain_right = None

    def parts(self):
        return [self.left, self.right]

    def cache_need(self):
        needs = []
        for side, m in (("left", self.left), ("right", self.right)):
            need = m.cache_need()
            for one in need if isinstance(need, (tuple, list)) else (need,):
                if isinstance(one, StateNeed):
                    one = StateNeed(tuple((f"{side}.{name}", shape, dt) for name, shape, dt in one.tensors))
                if one is not None:
                    needs.append(one)
        if sum(isinstance(n, KVNeed) for n in needs) > 1:
            raise ValueError("two mixers side by side that both read pages are not supported")
        return tuple(needs) if needs else None

    def param_specs(self):
        H = self.hidden_size
        return self.left.param_specs() + self.right.param_specs() + \
            [ParamSpec(self.names["left"], (H,), "vector"), ParamSpec(self.names["right"], (H,), "vector")]

    def load(self, fetch):
        self.left.load(fetch)
        self.right.load(fetch)
        self.w_in = torch.cat(self.left.input_weights() + self.right.input_weights(), dim=0).contiguous()
        self.left_width = sum(w.shape[0] for w in self.left.input_weights())
        # the two mixers read their matrices through the fused one only: drop the separate copies
        for m in (self.left, self.right):
            for attr in ("wqkv", "w_in"):
                if getattr(m, attr, None) is not None:
                    setattr(m, attr, None)
        self.gain_left, self.gain_right = fetch(self.names["left"]).contiguous(), fetch(self.names["right"]).contiguous()
        if self.gain_left.dtype != self.gain_right.dtype:
            self.gain_right = self.gain_right.to(self.gain_left.dtype)

    @staticmethod
    def _side(cache: CacheRef, side: str) -> CacheRef:
        names = {k[len(side) + 1:]: v for k, v in (cache.state_names or {}).items() if k.startswith(side + ".")}
        return CacheRef(cache.group, cache.layer, cache.writes, names or None)

    def __call__(self, x: torch.Tensor, ctx, cache: CacheRef):
        fused, parts = ops.project(x, self.w_in, lambda name, shape, dt: ctx.buffer("parallel_in_" + name, shape, dt))
        a = self.left.mix(fused, parts, 0, ctx, self._side(cache, "left"))
        b = self.right.mix(fused, parts, self.left_width, ctx, self._side(cache, "right"))
        # half the sum of the two normed outputs is taken by whoever reads the branch (the next norm's kernel)
        return MeanOfNormed(a, self.gain_left, b, self.gain_right, self.eps, 0.5)


@MIXERS.register("delta_rule")
class DeltaRule:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype: torch.dtype):
        self.heads, self.kv_heads = int(spec.num_heads), int(spec.num_kv_heads)
        self.dim, self.vdim, self.taps = int(spec.key_dim), int(spec.value_dim), int(spec.conv_taps)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads are no multiple of {self.kv_heads} query/key heads")
        if self.dim > 256 or self.vdim > 256 or not 1 <= self.taps <= 16:
            raise ValueError(f"key_dim {self.dim}, value_dim {self.vdim}, conv_taps {self.taps}: the kernels hold heads of up to 256 "
                             f"channels and convolutions of up to 16 taps")
        self.eps, self.unit_eps, self.q_scale = float(spec.eps), float(spec.unit_norm_eps), float(spec.options.get("q_scale", 1.0))
        self.hidden_size, self.model_dtype = hidden_size, model_dtype
        self.names = {k: spec.options[k] for k in ("q_proj", "k_proj", "v_proj", "g_proj", "o_proj", "q_conv", "k_conv", "v_conv",
                                                   "beta_proj", "decay_proj", "decay_log", "decay_bias", "head_norm_weight")}
        GD, HV = self.kv_heads * self.dim, self.heads * self.vdim
        self.offsets = {"q": 0, "k": GD, "v": 2 * GD, "g": 2 * GD + HV, "b": 2 * GD + 2 * HV, "a": 2 * GD + 2 * HV + self.heads}
        self.width = 2 * GD + 2 * HV + 2 * self.heads
        self.channels = 2 * GD + HV
        self.tag = ""
        self.w_in = self.wo = self.conv = self.a_log = self.dt_bias = self.norm_weight = None

    def cache_need(self):
        need = [("state", (self.heads, self.dim, self.vdim), torch.float32)]
        if self.taps > 1:
            need.append(("conv", (self.taps - 1, self.channels), torch.float32))
        return StateNeed(tuple(need))

    def param_specs(self):
        H, n, GD, HV = self.hidden_size, self.names, self.kv_heads * self.dim, self.heads * self.vdim
        return [ParamSpec(n["q_proj"], (GD, H)), ParamSpec(n["k_proj"], (GD, H)), ParamSpec(n["v_proj"], (HV, H)),
                ParamSpec(n["g_proj"], (HV, H)), ParamSpec(n["beta_proj"], (self.heads, H)), ParamSpec(n["decay_proj"], (self.heads, H)),
                ParamSpec(n["o_proj"], (H, HV)), ParamSpec(n["q_conv"], (GD, self.taps)), ParamSpec(n["k_conv"], (GD, self.taps)),
                ParamSpec(n["v_conv"], (HV, self.taps)), ParamSpec(n["decay_log"], (self.heads,), "vector"),
                ParamSpec(n["decay_bias"], (self.heads,), "vector"), ParamSpec(n["head_norm_weight"], (self.vdim,), "vector")]

    def load(self, fetch):
        n = self.names
        mats = [fetch(n[k]) for k in ("q_proj", "k_proj", "v_proj", "g_proj", "beta_proj", "decay_proj")]
        pad = -self.width % 8             # the product's rows in steps of 8 columns (16 bytes of the matrix type)
        if pad:
            mats.append(mats[0].new_zeros((pad, self.hidden_size)))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.wo = fetch(n["o_proj"]).contiguous()
        self.conv = [fetch(n[k]).contiguous() for k in ("q_conv", "k_conv", "v_conv")]
        self.a_log = fetch(n["decay_log"]).to(self.conv[0].dtype).contiguous()
        self.dt_bias = fetch(n["decay_bias"]).to(self.conv[0].dtype).contiguous()
        self.norm_weight = fetch(n["head_norm_weight"]).contiguous()

    def input_weights(self) -> list:
        return [self.w_in]

    def __call__(self, x: torch.Tensor, ctx, cache: CacheRef):
        fused, parts = ops.project(x, self.w_in, lambda name, shape, dt: ctx.buffer(self.tag + "delta_in_" + name, shape, dt))
        return self.mix(fused, parts, 0, ctx, cache)

    def mix(self, fused: torch.Tensor, parts: int, col0: int, ctx, cache: CacheRef):
        """The mixer on the columns from col0 of a fused product [n, W] (or partial sums [parts, n, W])."""
        n, H, G, D, V, f32 = fused.shape[-2], self.heads, self.kv_heads, self.dim, self.vdim, torch.float32
        off = {k: col0 + v for k, v in self.offsets.items()}
        q = ctx.buffer(self.tag + "delta_q", (n, G * D), f32)
        k = ctx.buffer(self.tag + "delta_k", (n, G * D), f32)
        v = ctx.buffer(self.tag + "delta_v", (n, H * V), f32)
        beta = ctx.buffer(self.tag + "delta_beta", (n, H), f32)
        decay = ctx.buffer(self.tag + "delta_decay", (n, H), f32)
        conv_state = ctx.state(cache.state_names["conv"]) if self.taps > 1 else None
        ops.delta_prepare(fused, parts, off, H, G, D, V, self.taps, *self.conv, self.a_log, self.dt_bias, ctx.token_req,
                          ctx.req_q_start, ctx.req_slot, conv_state, self.unit_eps, self.q_scale, q, k, v, beta, decay)
        ops.delta_conv_update(fused, parts, off, H, G, D, V, self.taps, ctx.req_q_start, ctx.req_q_len, ctx.req_slot, conv_state)
        o = ctx.buffer(self.tag + "delta_o", (n, H * V), f32)
        ops.delta_scan(q, k, v, beta, decay, ctx.state(cache.state_names["state"]), o, ctx.req_q_start, ctx.req_q_len, ctx.req_slot,
                       H, G, D, V)
        gated = ctx.buffer(self.tag + "delta_gated", (n, H * V), self.model_dtype)
        ops.head_gate_norm(o, fused, parts, off["g"], self.norm_weight, self.eps, gated, H, V)
        return as_branch(ops.project(gated, self.wo, lambda name, shape, dt: ctx.buffer(self.tag + "delta_out_" + name, shape, dt)))
