"""Zafilix as a plan of parts.

Every layer is a 'branch_normed' block: the sublayers read the residual as it is and a root-mean-square norm with a
gain of 1 + w stands behind each of them, x += norm1(mixer(x)), x += norm2(ff(x)).  The mixer is one of two.
*Attention*: grouped heads, value heads of their own size, q and k normed over their whole rows (all heads at once) in
front of a rotary turn of interleaved pairs whose frequencies are divided by a factor, a score scale of its own, a mask
of blocks (a position sees the earlier positions of its own block of `size` positions), and a sigmoid gate from the
mixer's input on the heads' outputs in front of the output projection.  *Latent attention*: one normed latent row and
one turned key part per position are all that is cached; every head's key and value are products of the latent row,
which the mixer folds into the queries and the outputs, so that attention runs over the cached rows themselves; a
sliding window.  The feed-forward is down(relu(up x)^2).  A layer may run on another layer's tensors with a cache of its
own.  The embedding is scaled, the head untied; its logits are scaled and pass a tanh cap.

Checkpoint names: embed, head, final.norm; layer i: l<i>.norm1 / norm2, l<i>.mix.q / k / v / g / o / q.norm / k.norm
(attention) or l<i>.mix.q / dkv / dkv.norm / uk / uv / o (latent attention), l<i>.mlp.up / down.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zafilix import ZafilixConfig
from ..parts import LayerRun, ModelPlan, spec

NO_POSITION_LIMIT = 1 << 30


def _rope(rot, size: int, pairing: str):
    rot = rot or {"dims": 0, "base": 1.0}
    factor = (rot.get("scaling") or {}).get("factor")
    return spec("rope", theta=rot["base"], head_dim=size, rotary_dim=rot["dims"], exact_table=True, pairing=pairing,
                frequency_divisor=factor)


def _attention(p: str, m: dict, eps: float):
    mask = m.get("mask") or {}
    return spec("attention", num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
                window=mask.get("size"), mask="blocks" if mask else "window", scale=m["scale"],
                row_norm={"q": p + "q.norm", "k": p + "k.norm", "eps": eps}, gate_proj=p + "g",
                position=_rope(m.get("rot"), m["dim"], "interleaved"),
                q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", o_proj=p + "o")


def _latent(p: str, m: dict, eps: float):
    mask = m.get("mask") or {}
    return spec("latent_attention", num_heads=m["heads"], plain_dim=m["dim"], rot_dim=m["rot_dim"], value_dim=m["vdim"],
                kv_rank=m["kv_rank"], scale=m["scale"], window=mask.get("size"), eps=eps,
                position=_rope(m.get("rot"), m["rot_dim"], "half"),
                q_proj=p + "q", down_proj=p + "dkv", latent_norm=p + "dkv.norm", up_k=p + "uk", up_v=p + "uv", o_proj=p + "o")


@register_architecture("Zafilix", ZafilixConfig)
def zafilix_plan(cfg: ZafilixConfig) -> ModelPlan:
    def norm(name):
        return spec("rmsnorm", weight=name, eps=cfg.eps, unit_offset=True)
    blocks, block_of, runs = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if cfg.owner(i) == i:
            p = f"l{i}."
            make = _attention if layer["type"] == "attention" else _latent
            options = dict(reader=spec("identity"), mixer=make(p + "mix.", layer["mixer"], cfg.eps), norm_mixer_out=norm(p + "norm1"))
            if layer["mlp"] is not None:
                options.update(feed_forward=spec("dense", intermediate_size=layer["mlp"]["ff"], activation="relu_squared",
                                                 up_proj=p + "mlp.up", down_proj=p + "mlp.down"),
                               norm_ff_out=norm(p + "norm2"))
            block_of[i] = len(blocks)
            blocks.append(spec("branch_normed", **options))
        runs.append(LayerRun(block_of[cfg.owner(i)]))
    return ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=NO_POSITION_LIMIT,
        embedding=spec("scaled_embedding", weight="embed", vocab_size=cfg.vocab, scale=cfg.embedding_scale),
        blocks=blocks, final_norm=norm("final.norm"),
        head=spec("logits_head", tied=False, weight="head", vocab_size=cfg.vocab, scale=cfg.logit_scale,
                  softcap=cfg.logit_softcap),
        runs=runs,
    )
