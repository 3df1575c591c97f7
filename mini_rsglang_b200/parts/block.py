"""How a layer's parts are arranged.  "pre_norm": x + mixer(norm1(x)), then
+ feed_forward(norm2(.)) (reference: crates/models/src/qwen3.rs:176-225).  "sandwich_norm": a norm before and after
each branch.  "parallel": both branches read one norm's output, x + (mixer(norm1(x)) + feed_forward(norm1(x))).

The residual stream is float32.  A branch's output is not added by a kernel of its own: it
is handed on as `pending`, and the next norm adds it while it reads the stream anyway; or,
with few rows, the branch's last product adds it and the norm rides on the products around it
(`Prenormed` in parts/base.py)."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Normed, Prenormed, ResidualLink, observing, plain


def _branch(part, h, stream, norm, *args):
    """Runs a mixer or feed-forward on `h`, telling it where its output goes if it can use that."""
    if isinstance(h, Prenormed) and not getattr(part, "takes_prenormed", False):
        h = plain(h)
    if getattr(part, "adds_to_stream", False) and norm is not None and getattr(norm, "rides_on_products", False):
        return part.forward(h, *args, into=ResidualLink(stream, norm))
    return part.forward(h, *args)


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    links_norms = True
    roles = {"norm1": NORMS, "mixer": MIXERS, "norm2": NORMS, "feed_forward": FEED_FORWARDS}
    optional_roles = ("norm2", "feed_forward")       # a layer may be a mixer alone (both are left out together)
    entry_role = "norm1"

    def __init__(self, prefix: str, **parts):
        super().__init__(prefix, **parts)
        if (self.norm2 is None) != (self.feed_forward is None):
            raise InvalidRequest(f"block at {prefix!r}: a feed-forward comes with the norm before it")

    def forward(self, stream, pending, ctx, cache, write_cache=True, next_norm=None):
        if observing(ctx):
            return self.forward_observed(stream, pending, ctx, cache, write_cache)
        h = self.norm1.add_norm(stream, pending)
        if self.feed_forward is None:
            return _branch(self.mixer, h, stream, next_norm, ctx, cache, write_cache)
        a = _branch(self.mixer, h, stream, self.norm2, ctx, cache, write_cache)
        h = self.norm2.add_norm(stream, a)
        return _branch(self.feed_forward, h, stream, next_norm, ctx)

    def forward_observed(self, stream, pending, ctx, cache, write_cache):
        """The same with every norm a kernel of its own and the reference's observer called on its labels
        (crates/models/src/qwen3.rs:177-226): input_norm here, the mixer's and feed-forward's inside them, output."""
        h = plain(self.norm1.add_norm(stream, pending))
        ctx.observe(f"{ctx.label}-input_norm", h)
        a = self.mixer.forward(h, ctx, cache, write_cache)
        if self.feed_forward is None:
            ctx.observe(f"{ctx.label}-output", stream + a.float())
            return a
        h = plain(self.norm2.add_norm(stream, a))
        f = self.feed_forward.forward(h, ctx)
        ctx.observe(f"{ctx.label}-output", stream + f.float())
        return f


@BLOCKS.register("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before and a norm after each branch: x <- x + m norm1b(mixer(norm1(x))), then, where the layer has a
    feed-forward, x <- x + m norm2b(feed_forward(norm2(x))); m = `branch_scale` (1 unless the layer's spec says otherwise).

    The branches' last products leave float32 sums; one kernel norms a branch's output, adds it to the float32
    stream and runs the norm that reads the stream next (`kernels.postnorm_add_norm`), so the sum and both
    statistics are float32 and a layer's four norms are two launches.  What follows the block's last branch is the
    next block's first norm: its rows are handed on as a `Normed`."""

    links_norms = True
    roles = {"norm1": NORMS, "mixer": MIXERS, "norm1b": NORMS, "norm2": NORMS, "feed_forward": FEED_FORWARDS, "norm2b": NORMS}
    optional_roles = ("norm2", "feed_forward", "norm2b")
    entry_role = "norm1"

    def __init__(self, prefix: str, branch_scale: float = 1.0, **parts):
        super().__init__(prefix, **parts)
        self.branch_scale = float(branch_scale)
        given = [self.parts.get(role) is not None for role in self.optional_roles]
        if any(given) and not all(given):
            raise InvalidRequest(f"block at {prefix!r}: a feed-forward comes with the norm before and the norm after it")
        for role in ("norm1b", "norm2", "norm2b"):
            norm = self.parts.get(role)
            if norm is not None and not getattr(norm, "rides_on_products", False):
                raise InvalidRequest(f"block at {prefix!r}: the norm {role!r} must be an RMS norm with float32 weights")

    def _join(self, stream, branch, post, following):
        """stream += branch_scale * post(branch); the rows of `following` (a norm, or None) over the sum."""
        fused = following is not None and getattr(following, "rides_on_products", False) and not following.gathers_rows
        if branch.dtype is not torch.float32:          # a branch written for another arrangement
            branch = branch.float()
        out = torch.empty(stream.shape, dtype=self.runtime.dtype, device=stream.device) if fused else None
        kernels.postnorm_add_norm(stream, branch, post.weight, post.eps, following.weight if fused else None,
                                  following.eps if fused else 0.0, out, self.branch_scale)
        return Normed(out, following, stream) if fused else None

    def forward(self, stream, pending, ctx, cache, write_cache=True, next_norm=None):
        h = plain(self.norm1.add_norm(stream, pending))
        if observing(ctx):
            ctx.observe(f"{ctx.label}-input_norm", h)
        a = self.mixer.forward(h, ctx, cache, write_cache)
        if self.feed_forward is None:
            pending = self._join(stream, a, self.norm1b, next_norm)
        else:
            h = self._join(stream, a, self.norm1b, self.norm2).rows
            f = self.feed_forward.forward(h, ctx)
            pending = self._join(stream, f, self.norm2b, next_norm)
        if observing(ctx):
            ctx.observe(f"{ctx.label}-output", stream.clone())
        return pending


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """Both branches side by side on one normed input: with h = norm1(x), x <- x + (mixer(h) + feed_forward(h)); a layer may
    be a mixer alone.

    The branches' last products leave float32 sums; one kernel adds both to the float32 stream and runs the norm that reads
    the stream next (`kernels.add_branches_norm`), whose rows are handed on as a `Normed`: a layer is one norm launch."""

    links_norms = True
    roles = {"norm1": NORMS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS}
    optional_roles = ("feed_forward",)
    entry_role = "norm1"

    def forward(self, stream, pending, ctx, cache, write_cache=True, next_norm=None):
        h = plain(self.norm1.add_norm(stream, pending))
        if observing(ctx):
            ctx.observe(f"{ctx.label}-input_norm", h)
        a = self.mixer.forward(h, ctx, cache, write_cache)
        f = self.feed_forward.forward(h, ctx) if self.feed_forward is not None else None
        if a.dtype is not torch.float32:          # a branch written for another arrangement
            a = a.float()
        if f is not None and f.dtype is not torch.float32:
            f = f.float()
        fused = next_norm is not None and getattr(next_norm, "rides_on_products", False) and not next_norm.gathers_rows
        out = torch.empty(stream.shape, dtype=self.runtime.dtype, device=stream.device) if fused else None
        kernels.add_branches_norm(stream, a, f, next_norm.weight if fused else None, next_norm.eps if fused else 0.0, out)
        if observing(ctx):
            ctx.observe(f"{ctx.label}-output", stream.clone())
        return Normed(out, next_norm, stream) if fused else None
