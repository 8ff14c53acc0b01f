"""How a layer's parts are wired (transformer.rs:20-48)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Arrangement
from .registry import register


@register("arrangement", "pre_norm")
class PreNorm(Arrangement):
    """h1 = x + mixer(norm(x)); h2 = h1 + ff(norm(h1)): the un-normalised stream is carried
    (transformer.rs:31-47).  Roles: mixer, feed_forward, mixer_norm, feed_forward_norm."""

    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def forward(self, residual, ctx, cache_layer, writes_cache):
        normed = ctx.buffer("normed", (residual.shape[0], residual.shape[1]), ctx.dtype)
        self.mixer_norm.forward(residual, normed)
        self.mixer.forward(normed, residual, ctx, cache_layer, writes_cache)
        if self.feed_forward is None:
            return
        self.feed_forward_norm.forward(residual, normed)
        self.feed_forward.forward(normed, residual, ctx)


@register("arrangement", "pre_norm_optional_ff")
class PreNormOptionalFeedForward(PreNorm):
    """The same for models whose layers may have no feed-forward (and then no norm for it)."""

    OPTIONAL = ("feed_forward", "feed_forward_norm")

    def __init__(self, **parts):
        super().__init__(**parts)
        if (self.feed_forward is None) != (self.feed_forward_norm is None):
            raise ValueError("pre_norm_optional_ff: a feed-forward comes with its norm, and the norm with it")


@register("arrangement", "parallel_two_norms")
class ParallelTwoNorms(Arrangement):
    """x <- x + mixer(norm_a(x)) + ff(norm_b(x)): mixer and feed-forward read the same stream, each
    through a norm of its own; both add onto the float32 stream.  A layer may have no feed-forward
    (then it has no second norm either)."""

    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}
    OPTIONAL = ("feed_forward", "feed_forward_norm")

    def forward(self, residual, ctx, cache_layer, writes_cache):
        shape = (residual.shape[0], residual.shape[1])
        normed = ctx.buffer("normed", shape, ctx.dtype)
        if self.feed_forward is not None:
            # both norms read the stream before either branch adds to it (small steps: one kernel for the two)
            normed_ff = ctx.buffer("normed_ff", shape, ctx.dtype)
            pair = getattr(self.mixer_norm, "forward_with", None)
            if pair is None or not pair(self.feed_forward_norm, residual, normed, normed_ff):
                self.mixer_norm.forward(residual, normed)
                self.feed_forward_norm.forward(residual, normed_ff)
        else:
            self.mixer_norm.forward(residual, normed)
        self.mixer.forward(normed, residual, ctx, cache_layer, writes_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(normed_ff, residual, ctx)


@register("arrangement", "parallel_shared_norm")
class ParallelSharedNorm(Arrangement):
    """x <- x + (mixer(h) + ff(h)) with h = norm(x): one norm, and mixer and feed-forward both read its
    output; both add onto the float32 stream.  A layer may have no feed-forward."""

    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm": "norm"}
    OPTIONAL = ("feed_forward",)

    def forward(self, residual, ctx, cache_layer, writes_cache):
        normed = ctx.buffer("normed", (residual.shape[0], residual.shape[1]), ctx.dtype)
        self.norm.forward(residual, normed)
        self.mixer.forward(normed, residual, ctx, cache_layer, writes_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(normed, residual, ctx)


@register("arrangement", "pre_post_norm")
class PrePostNorm(Arrangement):
    """x <- x + post_a(mixer(pre_a(x))), then x <- x + post_b(ff(pre_b(x))): every sublayer is normalised going in and
    coming out.  The sublayer writes into a zeroed float32 buffer of its own instead of the stream, so that its result
    can be normalised before it joins.  A layer may have no feed-forward (and then no norms for it), and may have a
    `depth` part that turns the layer's result into what goes on to the next layer.

    With norms that need no statistics of a row (`fused()`), joining the stream, the sum over depth and the next
    sublayer's norm are one elementwise pass (`ops.stream_update`); any other norm takes the steps one by one."""

    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "mixer_post_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward_post_norm": "norm", "depth": "depth"}
    OPTIONAL = ("feed_forward", "feed_forward_norm", "feed_forward_post_norm", "depth")

    def __init__(self, **parts):
        super().__init__(**parts)
        if (self.feed_forward is None) != (self.feed_forward_norm is None) or \
                (self.feed_forward is None) != (self.feed_forward_post_norm is None):
            raise ValueError("pre_post_norm: a feed-forward comes with its two norms, and they with it")

    @staticmethod
    def _join(stream, branch, post, ctx, depth=None, then=None, then_out=None):
        """stream += post(branch); branch <- 0; the sum over depth; then_out = then(stream)."""
        post_f = getattr(post, "fused", None)
        then_f = getattr(then, "fused", None) if then is not None else None
        depth_kw = depth.fused(ctx, stream) if depth is not None else None
        if post_f is not None and (then is None or then_f is not None) and (depth is None or depth_kw is not None):
            ops.stream_update(stream, branch=branch, post=post_f(), next_norm=then_f() if then is not None else None,
                              next_out=then_out, **(depth_kw or {}))
            return
        normed = ctx.buffer("branch_normed", tuple(stream.shape), torch.float32)
        post.forward(branch, normed)
        branch.zero_()
        ops.stream_update(stream, branch=normed)
        if depth is not None:
            depth.leave(stream, ctx)
        if then is not None:
            then.forward(stream, then_out)

    def forward(self, residual, ctx, cache_layer, writes_cache):
        shape = (residual.shape[0], residual.shape[1])
        normed = ctx.buffer("normed", shape, ctx.dtype)
        branch = ctx.zeroed_buffer("branch", shape, torch.float32)
        if self.depth is not None:
            self.depth.enter(residual, ctx)
        self.mixer_norm.forward(residual, normed)
        self.mixer.forward(normed, branch, ctx, cache_layer, writes_cache)
        if self.feed_forward is None:
            self._join(residual, branch, self.mixer_post_norm, ctx, depth=self.depth)
            return
        self._join(residual, branch, self.mixer_post_norm, ctx, then=self.feed_forward_norm, then_out=normed)
        self.feed_forward.forward(normed, branch, ctx)
        self._join(residual, branch, self.feed_forward_post_norm, ctx, depth=self.depth)
