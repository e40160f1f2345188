"""Arrangements of a mixer, a feed-forward and norms around the residual stream.

`SandwichBlock` is Gemma2's (`gemma/gemma.go:162-167`): a norm before and a
norm after each sublayer, the second applied to the sublayer's output before it
is added:  r = Mixer(N_in(x)); h = x + N_post_mixer(r); r = FF(N_pre_ff(h));
out = h + N_post_ff(r).

`PreNormBlock` is the usual arrangement without the norms after the sublayers
(`qwen/block.go:58-61`): h = x + Mixer(N_in(x)); out = h + FF(N_pre_ff(h)).

The residual stream is float32 and is updated in place.  A block may be handed
its first norm's output (computed by the block before it together with that
block's last residual sum) and may be asked to apply the next block's first
norm to its own result, which saves a pass over the stream per layer.
"""
from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm, StepContext
from .norm import plain_residual_add


class SandwichBlock(Block):
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, input_norm: Norm, post_mixer_norm: Norm,
                 pre_ff_norm: Norm, post_ff_norm: Norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.first_norm = input_norm
        self.post_mixer_norm, self.pre_ff_norm, self.post_ff_norm = post_mixer_norm, pre_ff_norm, post_ff_norm

    def sub_parts(self):
        return [self.first_norm, self.mixer, self.post_mixer_norm, self.pre_ff_norm, self.feed_forward,
                self.post_ff_norm]

    def forward(self, h, ctx: StepContext, line, y_in=None, next_norm: Norm | None = None):
        T, H = h.shape
        dt = ctx.rt.dtype
        y = y_in if y_in is not None else self.first_norm.forward(h, ctx, ctx.ws.buf("block.y", (T, H), dt))
        r = self.mixer.forward(y, ctx, line)
        y = self.post_mixer_norm.residual_add(h, r, ctx, self.pre_ff_norm, ctx.ws.buf("block.y", (T, H), dt))
        r = self.feed_forward.forward(y, ctx)
        y_next = self.post_ff_norm.residual_add(h, r, ctx, next_norm,
                                                ctx.ws.buf("block.y", (T, H), dt) if next_norm is not None else None)
        return h, y_next


class PreNormBlock(Block):
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, input_norm: Norm, pre_ff_norm: Norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.first_norm = input_norm
        self.pre_ff_norm = pre_ff_norm

    def sub_parts(self):
        return [self.first_norm, self.mixer, self.pre_ff_norm, self.feed_forward]

    def forward(self, h, ctx: StepContext, line, y_in=None, next_norm: Norm | None = None):
        T, H = h.shape
        dt = ctx.rt.dtype
        y = y_in if y_in is not None else self.first_norm.forward(h, ctx, ctx.ws.buf("block.y", (T, H), dt))
        r = self.mixer.forward(y, ctx, line)
        y = plain_residual_add(h, r, ctx, self.pre_ff_norm, ctx.ws.buf("block.y", (T, H), dt))
        r = self.feed_forward.forward(y, ctx)
        y_next = plain_residual_add(h, r, ctx, next_norm,
                                    ctx.ws.buf("block.y", (T, H), dt) if next_norm is not None else None)
        return h, y_next
