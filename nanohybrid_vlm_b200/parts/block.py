"""Pre-norm block with the residual carried apart (nanovllm/models/qwen3.py:146-159).

Every sub-block's output is added to the residual stream inside the next norm, so the
block hands on (output of its feed-forward, residual) and the model's final norm does the
last add.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import BLOCKS, FEED_FORWARDS, FILTERS, MIXERS, NORMS, Block, CompositeNeed, Pending


class PreNormResidualBlock(Block):
    def forward(self, hidden, residual, batch, cache):
        if residual is None:
            residual = hidden
            x = self.mixer_norm.forward(hidden)
        else:
            x = self.mixer_norm.forward_add(hidden, residual)
        a = self.mixer.forward(x, batch, cache)
        x = self.ffn_norm.forward_add(a, residual)
        m = self.ffn.forward(x, batch)
        return m, residual


class ParallelResidualBlock(Block):
    """One norm whose output both the mixer and the feed-forward read: x <- x + mult * (mixer(h) + ffn(h)) with
    h = norm(x).  The residual stream x is kept in float32: the block hands on its sub-blocks' outputs as a
    :class:`Pending` (each with its factor) and the next norm (the next layer's, or the model's last) adds them in
    32-bit.  Parameter: ``residual_mult``.  A layer may have no feed-forward.

    Optional input filters (``mixer_filter``, ``ffn_filter``; registry FILTERS): what each sub-block reads is then the
    filter's output over h.  Both filters read the same h, so the block keeps ONE state for them (the filter's
    ``state_need``) beside what the mixer keeps: the layer's need is the composite (filter state, mixer's need), and
    the mixer gets its child view."""
    SLOTS = {"mixer": MIXERS, "norm": NORMS, "ffn": FEED_FORWARDS, "mixer_filter": FILTERS, "ffn_filter": FILTERS}
    OPTIONAL = ("ffn", "mixer_filter", "ffn_filter")

    def __init__(self, spec, parts):
        super().__init__(spec, parts)
        self.mult = float(spec.get("residual_mult", 1.0))
        self.filters = [parts.get("mixer_filter"), parts.get("ffn_filter") if "ffn" in parts else None]
        if "ffn_filter" in parts and "ffn" not in parts:
            raise ValueError("a filter in front of the feed-forward needs a feed-forward")
        both = [f for f in self.filters if f is not None]
        if len(both) == 2 and both[0].state_need() != both[1].state_need():
            raise ValueError("the two input filters of a block share one state: their sizes must agree")
        self.filtered = bool(both)

    def cache_need(self):
        need = super().cache_need()
        if not self.filtered:
            return need
        return CompositeNeed((next(f for f in self.filters if f is not None).state_need(), need))

    def forward(self, hidden, residual, batch, cache):
        if residual is None:
            residual = hidden if hidden.dtype == torch.float32 else hidden.float()
            hidden = Pending()
        x = self.norm.forward_add(hidden, residual)
        xm = xf = x
        if self.filtered:
            kept, cache = cache.children
            fm, ff = self.filters
            if fm is not None and ff is not None:
                xm, xf = fm.forward_pair(ff, x, batch, kept.state)
            elif fm is not None:
                xm = fm.forward(x, batch, kept.state)
            else:
                xf = ff.forward(x, batch, kept.state)
        terms = [(t, self.mult * c) for t, c in self.mixer.forward_terms(xm, batch, cache)]
        ffn = self.parts.get("ffn")
        if ffn is not None:
            terms.append((ffn.forward(xf, batch), self.mult))
        return Pending(tuple(terms)), residual


class SandwichResidualBlock(Block):
    """A norm before and after each sub-block: x <- x + post1(mixer(pre1(x))), then x <- x + post2(ffn(pre2(x))).  The
    residual stream x is kept in float32.  A sub-block's output is handed on as a :class:`Pending` together with the
    norm it still has to pass; the next norm in line (this layer's second pre-norm, the next layer's first, or the
    model's last) applies that norm, adds the result in 32-bit and norms the sum, in one kernel where the norms allow it.
    A layer may have no feed-forward (then also neither of its norms)."""
    SLOTS = {"mixer": MIXERS, "mixer_norm": NORMS, "mixer_post_norm": NORMS, "ffn": FEED_FORWARDS, "ffn_norm": NORMS,
             "ffn_post_norm": NORMS}
    OPTIONAL = ("ffn", "ffn_norm", "ffn_post_norm")

    def __init__(self, spec, parts):
        super().__init__(spec, parts)
        has = [name in parts for name in self.OPTIONAL]
        if any(has) and not all(has):
            raise ValueError("a feed-forward comes with both of its norms, or not at all")

    def forward(self, hidden, residual, batch, cache):
        if residual is None:
            residual = hidden if hidden.dtype == torch.float32 else hidden.float()
            hidden = Pending()
        x = self.mixer_norm.forward_add(hidden, residual)
        pending = Pending(((self.mixer.forward(x, batch, cache), 1.0),), post=self.mixer_post_norm)
        ffn = self.parts.get("ffn")
        if ffn is not None:
            x = self.ffn_norm.forward_add(pending, residual)
            pending = Pending(((ffn.forward(x, batch), 1.0),), post=self.ffn_post_norm)
        return pending, residual


class PostNormResidualBlock(Block):
    """A norm on each sub-block's output only: x <- x + post1(mixer(x)), then x <- x + post2(ffn(x)).  The sub-blocks
    read the stream x itself (rounded to the model's type); the stream is kept in float32.  Each norm (``mixer_norm``,
    ``ffn_norm``) norms its sub-block's output, multiplies it by its weight and, if it has one, by its scale per channel
    (``post_scale``), and adds the result onto the stream in one kernel (``Norm.add_normed``) that also hands back the
    new stream rounded, which the next sub-block reads.  A mixer whose output is a sum of terms that each pass a norm of
    their own (``forward_normed_terms``) has those norms done in the same kernel.  A layer may have no feed-forward
    (then also no second norm).  The block hands on an empty :class:`Pending` that carries the rounded stream."""
    OPTIONAL = ("ffn", "ffn_norm")

    def __init__(self, spec, parts):
        super().__init__(spec, parts)
        if ("ffn" in parts) != ("ffn_norm" in parts):
            raise ValueError("a feed-forward comes with its norm, or not at all")

    def forward(self, hidden, residual, batch, cache):
        if residual is None:
            residual = hidden if hidden.dtype == torch.float32 else hidden.float()
            hidden = Pending()
        if not isinstance(hidden, Pending) or hidden.terms:
            raise TypeError("this block follows blocks that leave nothing pending on a float32 stream")
        exact = self.mixer.env.dtype == torch.float32       # the stream itself is what the sub-blocks read
        x = residual if exact else hidden.rounded
        if x is None:
            x = self.mixer.new(*residual.shape)
            ops.stream_round(x, residual)
        terms = self.mixer.forward_normed_terms(x, batch, cache)
        x = self.mixer_norm.add_normed(terms, residual, getattr(self.mixer, "side_eps", None), want_rounded=not exact)
        ffn = self.parts.get("ffn")
        if ffn is not None:
            m = ffn.forward(residual if exact else x, batch)
            x = self.ffn_norm.add_normed(((m, 1.0, None),), residual, want_rounded=not exact)
        return Pending(rounded=x), residual


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
BLOCKS.register("postnorm_residual", PostNormResidualBlock)
BLOCKS.register("sandwich_residual", SandwichResidualBlock)
BLOCKS.register("parallel_residual", ParallelResidualBlock)
