"""Gudarax as a plan of parts.

Every layer is a pre-norm block of root-mean-square norms (plain gains): x += mixer(norm1(x)), x += ff(norm2(x)), and then a
*token input*: the layer's columns of a table row of the token itself, multiplied by gelu_tanh of a small projection of x,
projected back to the model width, root-mean-square normed and added.  The mixer is one of three.
*Attention*: grouped heads with values of their own size, biases on q, k and v, q and k normed over their whole rows (all
heads at once), no turn; a score loses slope_h * (i - j) with slope_h = 2^(-8 (h + 1) / heads); a sliding window; from the second
layer that says `v_mix` on, the values are blended with the first such layer's values of the same token before they are
cached.  *Latent attention*: queries through a normed latent row, keys and values as maps of one cached normed latent
row, every earlier key visible, a sigmoid gate from the mixer's input on the heads' outputs.  *Delta*: the gated delta
rule over a matrix state per head, fed through short convolutions.  The feed-forward is a gated SiLU unit, or routed
experts (sigmoid scores, the chosen experts' scores multiply their inputs, experts down(relu(up x)^2)).  The embedding is
scaled and a learned position row is added; the head is untied.

Checkpoint names: embed, pos, side.embed, head, final.norm; layer i: l<i>.norm1 / norm2, l<i>.side.gate / proj / norm,
l<i>.mix.q / k / v (+ .b) / q.norm / k.norm / vmix / o (attention), l<i>.mix.dq / dq.norm / uq / dkv / dkv.norm / uk / uv /
g / o (latent attention), l<i>.mix.q / k / v (+ .conv) / b / a / A_log / dt_bias / norm / g / o (delta),
l<i>.mlp.gate / up / down or l<i>.mlp.router, l<i>.mlp.e<j>.up / down.
"""
from __future__ import annotations

from ..config.gudarax import GudaraxConfig
from ..config.registry import register_architecture
from ..parts import LayerRun, ModelPlan, spec

SLOPE_EXPONENT = 8.0          # head h of H loses 2^(-SLOPE_EXPONENT (h + 1) / H) a position of distance
UNIT_NORM_EPS = 1e-6          # q and k heads of the delta rule: x / sqrt(sum(x^2) + UNIT_NORM_EPS)


def distance_slopes(heads: int) -> list:
    return [2.0 ** (-SLOPE_EXPONENT * (h + 1) / heads) for h in range(heads)]


def _attention(p: str, m: dict, eps: float, mix_role):
    mask = m.get("mask") or {}
    return spec("attention", num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
                window=mask.get("size"), scale=m["scale"], row_norm={"q": p + "q.norm", "k": p + "k.norm", "eps": eps},
                bias={"q": p + "q.b", "k": p + "k.b", "v": p + "v.b"}, distance_slopes=distance_slopes(m["heads"]),
                value_mix=None if mix_role is None else {"weight": p + "vmix", "role": mix_role, "key": "value_mix"},
                position=spec("rope", theta=1.0, head_dim=m["dim"], rotary_dim=0, exact_table=True, pairing="half"),
                q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", o_proj=p + "o")


def _latent(p: str, m: dict, eps: float):
    return spec("latent_attention", num_heads=m["heads"], plain_dim=m["dim"], rot_dim=0, value_dim=m["vdim"],
                kv_rank=m["kv_rank"], scale=m["scale"], window=None, eps=eps,
                position=spec("rope", theta=1.0, head_dim=0, rotary_dim=0, exact_table=True, pairing="half"),
                query_latent={"rank": m["q_rank"], "down": p + "dq", "norm": p + "dq.norm", "up": p + "uq"}, gate_proj=p + "g",
                down_proj=p + "dkv", latent_norm=p + "dkv.norm", up_k=p + "uk", up_v=p + "uv", o_proj=p + "o")


def _delta(p: str, m: dict, eps: float):
    return spec("delta_rule", num_heads=m["heads"], num_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                conv_taps=m["conv"], eps=eps, unit_norm_eps=UNIT_NORM_EPS, q_scale=float(m["dim"]) ** -0.5,
                q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", q_conv=p + "q.conv", k_conv=p + "k.conv", v_conv=p + "v.conv",
                beta_proj=p + "b", decay_proj=p + "a", decay_log=p + "A_log", decay_bias=p + "dt_bias",
                head_norm_weight=p + "norm", g_proj=p + "g", o_proj=p + "o")


def _feed_forward(p: str, mlp: dict):
    if mlp["kind"] == "dense":
        return spec("gated_dense", intermediate_size=mlp["ff"], activation="silu", gate_proj=p + "gate", up_proj=p + "up",
                    down_proj=p + "down")
    return spec("routed_experts", num_experts=mlp["router"]["experts"], top=mlp["router"]["top"], router=p + "router",
                expert_prefix=p + "e", intermediate_size=mlp["expert"]["ff"], activation="relu_squared", scores="sigmoid",
                gated=False, weight_on="input")


@register_architecture("Gudarax", GudaraxConfig)
def gudarax_plan(cfg: GudaraxConfig) -> ModelPlan:
    def norm(name):
        return spec("rmsnorm", weight=name, eps=cfg.eps)
    blocks, mixing = [], False
    layers = len(cfg.layers)
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            role = None
            if m.get("v_mix"):
                role, mixing = ("later" if mixing else "first"), True
            mixer = _attention(p + "mix.", m, cfg.eps, role)
        elif layer["type"] == "latent_attention":
            mixer = _latent(p + "mix.", m, cfg.eps)
        else:
            mixer = _delta(p + "mix.", m, cfg.eps)
        options = dict(norm_in=norm(p + "norm1"), mixer=mixer)
        if layer["mlp"] is not None:
            options.update(norm_post=norm(p + "norm2"), feed_forward=_feed_forward(p + "mlp.", layer["mlp"]))
        if cfg.side_dim is not None:
            options.update(token_input=spec("token_gated_table", table="side.embed", vocab_size=cfg.vocab,
                                            table_width=layers * cfg.side_dim, first_column=i * cfg.side_dim, dim=cfg.side_dim,
                                            activation="gelu_tanh", gate_proj=p + "side.gate", out_proj=p + "side.proj"),
                           token_input_norm=norm(p + "side.norm"), reader=spec("identity"))
        blocks.append(spec("pre_norm", **options))
    return ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=spec("scaled_embedding", weight="embed", vocab_size=cfg.vocab, scale=cfg.embedding_scale,
                       position_table="pos", max_positions=cfg.max_positions),
        blocks=blocks, final_norm=norm("final.norm"),
        head=spec("logits_head", tied=False, weight="head", vocab_size=cfg.vocab),
        runs=[LayerRun(i) for i in range(layers)],
    )
