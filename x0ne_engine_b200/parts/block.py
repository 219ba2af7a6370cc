"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from .base import BLOCKS, Block
from .norm import PostNormed


class PreNormBlock(Block):
    """x += mixer(norm(x)); x += ffn(norm(x)).  The residual stays in float32; each add is fused
    into the norm that follows it, so a block takes the previous block's pending delta and
    returns its own (x0ne-core/runtime/src/engine.rs:749,781,823)."""
    replayable = True
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}

    def forward(self, ctx, entry, resid, delta, cache_entry=None, write_cache=True):
        normed = ctx.ws.buffer("normed", (ctx.ws.max_rows, resid.shape[-1]), ctx.dtype)
        self.mixer_norm.add_norm(ctx, resid, delta, normed, ctx.n_rows)
        delta = self.mixer.forward(ctx, entry, normed, ctx.n_rows, cache_entry=cache_entry, write_cache=write_cache)
        self.ffn_norm.add_norm(ctx, resid, delta, normed, ctx.n_rows)
        return self.ffn.forward(ctx, normed, ctx.n_rows)


class PreNormMixerBlock(Block):
    """x += mixer(norm(x)) and nothing else: a pre-norm layer without a feed-forward."""
    replayable = True
    ROLES = {"mixer_norm": "norm", "mixer": "mixer"}

    def forward(self, ctx, entry, resid, delta, cache_entry=None, write_cache=True):
        normed = ctx.ws.buffer("normed", (ctx.ws.max_rows, resid.shape[-1]), ctx.dtype)
        self.mixer_norm.add_norm(ctx, resid, delta, normed, ctx.n_rows)
        return self.mixer.forward(ctx, entry, normed, ctx.n_rows, cache_entry=cache_entry, write_cache=write_cache)


class ParallelBlock(Block):
    """x += mixer(norm(x)) + ffn(norm(x)): one norm, both branches read its output, and their results
    are summed in float32 as they are added to the residual.  The add is again fused into the next
    norm, so the block hands on both results as a pair.  A layer may leave the feed-forward out."""
    replayable = True
    ROLES = {"norm": "norm", "mixer": "mixer", "ffn": "feed_forward"}
    OPTIONAL = ("ffn",)

    def __init__(self, parts):
        super().__init__(parts)
        if self.ffn is not None:
            self.ffn.out_buffer = "ffn.delta"       # beside the mixer's result, not over it

    def forward(self, ctx, entry, resid, delta, cache_entry=None, write_cache=True):
        normed = ctx.ws.buffer("normed", (ctx.ws.max_rows, resid.shape[-1]), ctx.dtype)
        self.norm.add_norm(ctx, resid, delta, normed, ctx.n_rows)
        mixed = self.mixer.forward(ctx, entry, normed, ctx.n_rows, cache_entry=cache_entry, write_cache=write_cache)
        if self.ffn is None:
            return mixed
        return (mixed, self.ffn.forward(ctx, normed, ctx.n_rows))


class SandwichBlock(Block):
    """x += post_norm(mixer(norm(x))); x += post_norm(ffn(norm(x))): every sublayer has a norm before it and one
    after it, on its result, before the add.  The normed result is never stored: the result travels with its
    norm (`PostNormed`) to the next norm in line, whose kernel norms it, adds it to the float32 residual
    and norms the sum.  A layer may leave the feed-forward (and its two norms) out."""
    replayable = True
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm", "ffn_norm": "norm", "ffn": "feed_forward",
             "ffn_post_norm": "norm"}
    OPTIONAL = ("ffn_norm", "ffn", "ffn_post_norm")

    def __init__(self, parts):
        super().__init__(parts)
        if (self.ffn is None) != (self.ffn_norm is None) or (self.ffn is None) != (self.ffn_post_norm is None):
            raise ValueError("a sandwich layer has its feed-forward with both of its norms, or none of the three")

    def forward(self, ctx, entry, resid, delta, cache_entry=None, write_cache=True):
        normed = ctx.ws.buffer("normed", (ctx.ws.max_rows, resid.shape[-1]), ctx.dtype)
        self.mixer_norm.add_norm(ctx, resid, delta, normed, ctx.n_rows)
        mixed = PostNormed(self.mixer.forward(ctx, entry, normed, ctx.n_rows, cache_entry=cache_entry, write_cache=write_cache),
                           self.mixer_post_norm)
        if self.ffn is None:
            return mixed
        self.ffn_norm.add_norm(ctx, resid, mixed, normed, ctx.n_rows)
        return PostNormed(self.ffn.forward(ctx, normed, ctx.n_rows), self.ffn_post_norm)


BLOCKS.register("prenorm", PreNormBlock)
BLOCKS.register("prenorm_mixer", PreNormMixerBlock)
BLOCKS.register("sandwich", SandwichBlock)
BLOCKS.register("parallel", ParallelBlock)
