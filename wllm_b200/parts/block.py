"""Arrangements of norms, mixer and feed-forward around the residual stream.

'pre_norm' (Gemma 1, src/wllm/models/gemma.py:83-93):
    x = x + mixer(norm_in(x));  x = x + feed_forward(norm_post(x))
A branch's output is left pending on the residual and folded in by the next norm
(the next block's, or the model's final one).

`feed_forward` may be absent: the block then has its first sublayer only.  With `token_input` the block ends with a
third addend that reads the residual as it then stands (through `reader`, kind 'identity') and the step's token ids, and
joins the residual through a norm of its own, x = x + token_input_norm(token_input(x, tokens)); it stays pending as a
`NormedBranch`, so the next norm of the residual runs that norm, the add and itself in one kernel.

spec options: norm_in, mixer, and norm_post, feed_forward (both or none), and token_input, token_input_norm, reader (all three or none).

'sandwich': a norm in front of and behind each sublayer,
    x = x + norm_mixer_out(mixer(norm_in(x)));  x = x + norm_ff_out(feed_forward(norm_post(x)))
The norm behind a sublayer acts on the branch alone; it is left pending on the residual as a `NormedBranch`, and the
next norm of the residual runs it, the add and itself in one kernel (`norm.branch` does it alone where that cannot be).  `feed_forward` may be None: the block then has its first sublayer only.

spec options: norm_in, mixer, norm_mixer_out, and norm_post, feed_forward, norm_ff_out (all three or none).

'branch_normed': a norm behind each sublayer and none in front; the sublayers read the residual as it is,
    x = x + norm_mixer_out(mixer(x));  x = x + norm_ff_out(feed_forward(x))
`reader` is the part that hands the residual to a sublayer (kind 'identity': the pending branch's norm, the add and the
rounding to the model's element type in one kernel).  `feed_forward` may be None.

spec options: reader, mixer, norm_mixer_out, and feed_forward, norm_ff_out (both or none).
"""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, CacheRef, NormedBranch, Residual


@BLOCKS.register("pre_norm")
class PreNormBlock:
    graph_safe = True
    def __init__(self, spec, hidden_size: int, model_dtype):
        kw = dict(hidden_size=hidden_size, model_dtype=model_dtype)
        self.norm_in = NORMS.build(spec.norm_in, **kw)
        self.mixer = MIXERS.build(spec.mixer, **kw)
        self.feed_forward = self.token_input = None
        if spec.options.get("feed_forward") is not None:
            self.norm_post = NORMS.build(spec.norm_post, **kw)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, **kw)
        if spec.options.get("token_input") is not None:
            self.reader = NORMS.build(spec.reader, **kw)
            self.token_input = FEED_FORWARDS.build(spec.token_input, **kw)
            self.token_input_norm = NORMS.build(spec.token_input_norm, **kw)

    def parts(self):
        out = [self.norm_in, self.mixer]
        if self.feed_forward is not None:
            out += [self.norm_post, self.feed_forward]
        if self.token_input is not None:
            out += [self.reader, self.token_input, self.token_input_norm]
        return out

    def cache_need(self):
        return self.mixer.cache_need()

    def __call__(self, residual: Residual, ctx, cache: CacheRef) -> None:
        residual.pending = self.mixer(self.norm_in(residual, ctx), ctx, cache)
        if self.feed_forward is not None:
            residual.pending = self.feed_forward(self.norm_post(residual, ctx), ctx)
        if self.token_input is not None:
            residual.pending = NormedBranch(self.token_input(self.reader(residual, ctx), ctx), self.token_input_norm)


@BLOCKS.register("sandwich")
class SandwichBlock:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype):
        kw = dict(hidden_size=hidden_size, model_dtype=model_dtype)
        self.norm_in = NORMS.build(spec.norm_in, **kw)
        self.mixer = MIXERS.build(spec.mixer, **kw)
        self.norm_mixer_out = NORMS.build(spec.norm_mixer_out, **kw)
        self.feed_forward = None
        if spec.options.get("feed_forward") is not None:
            self.norm_post = NORMS.build(spec.norm_post, **kw)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, **kw)
            self.norm_ff_out = NORMS.build(spec.norm_ff_out, **kw)

    def parts(self):
        first = [self.norm_in, self.mixer, self.norm_mixer_out]
        return first if self.feed_forward is None else first + [self.norm_post, self.feed_forward, self.norm_ff_out]

    def cache_need(self):
        return self.mixer.cache_need()

    def __call__(self, residual: Residual, ctx, cache: CacheRef) -> None:
        # the norm behind a sublayer is left to the next norm of the residual, which runs it inside its own kernel
        residual.pending = NormedBranch(self.mixer(self.norm_in(residual, ctx), ctx, cache), self.norm_mixer_out)
        if self.feed_forward is not None:
            residual.pending = NormedBranch(self.feed_forward(self.norm_post(residual, ctx), ctx), self.norm_ff_out)


@BLOCKS.register("branch_normed")
class BranchNormedBlock:
    graph_safe = True

    def __init__(self, spec, hidden_size: int, model_dtype):
        kw = dict(hidden_size=hidden_size, model_dtype=model_dtype)
        self.reader = NORMS.build(spec.reader, **kw)
        self.mixer = MIXERS.build(spec.mixer, **kw)
        self.norm_mixer_out = NORMS.build(spec.norm_mixer_out, **kw)
        self.feed_forward = None
        if spec.options.get("feed_forward") is not None:
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, **kw)
            self.norm_ff_out = NORMS.build(spec.norm_ff_out, **kw)

    def parts(self):
        first = [self.reader, self.mixer, self.norm_mixer_out]
        return first if self.feed_forward is None else first + [self.feed_forward, self.norm_ff_out]

    def cache_need(self):
        return self.mixer.cache_need()

    def __call__(self, residual: Residual, ctx, cache: CacheRef) -> None:
        residual.pending = NormedBranch(self.mixer(self.reader(residual, ctx), ctx, cache), self.norm_mixer_out)
        if self.feed_forward is not None:
            residual.pending = NormedBranch(self.feed_forward(self.reader(residual, ctx), ctx), self.norm_ff_out)
