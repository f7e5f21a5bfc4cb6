"""Two mixers side by side on the same input: out = left_scale * left(x) + right_scale * right(x).

Parameters: ``left`` and ``right`` (PartSpecs of registered mixers), ``left_scale``, ``right_scale``,
``prefixes`` (where each side's tensors sit under this part's own prefix; default ("left.", "right.")),
``side_norm_eps`` (a number: each side's output first passes an RMS norm over the model width with a weight of its
own, ``<prefix>out``, and this eps; None, the default: no such norms).
Each side keeps its own cache or state: the need is the composite of both, and each side gets its child view.
A block that adds weighted terms in 32-bit (``forward_terms``) receives the two outputs with their scales and no
sum is rounded on the way; ``forward`` gives the one summed tensor.
"""
from __future__ import annotations

from dataclasses import replace

from ..kernels import ops
from .base import MIXERS, CompositeNeed, Mixer
from .spec import ParamDecl


class ParallelMixers(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.sides = [MIXERS.get(spec[name].kind)(spec[name], env) for name in ("left", "right")]
        self.scales = (float(spec.get("left_scale", 1.0)), float(spec.get("right_scale", 1.0)))
        self.prefixes = tuple(spec.get("prefixes", ("left.", "right.")))
        eps = spec.get("side_norm_eps")
        self.side_eps = None if eps is None else float(eps)

    def params(self):
        decls = []
        for side, prefix in zip(self.sides, self.prefixes):
            for d in side.params():
                srcs = tuple(replace(s, name=prefix + s.name) for s in d.resolved_sources())
                decls.append(replace(d, name=prefix + d.name, sources=srcs))
            if self.side_eps is not None:
                if any(d.name == "out" for d in side.params()):
                    raise ValueError("a side of the pair owns a tensor named 'out', the name of its output norm's weight")
                decls.append(ParamDecl(prefix + "out", (self.env.hidden_size,), init="norm"))
        return decls

    def bind(self, tensors):
        self.side_weights = [None, None]
        for i, (side, prefix) in enumerate(zip(self.sides, self.prefixes)):
            mine = {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}
            if self.side_eps is not None:
                self.side_weights[i] = mine.pop("out")
            side.bind(mine)

    def cache_need(self):
        return CompositeNeed(tuple(side.cache_need() for side in self.sides))

    def streamed_weights(self):
        return [w for side in self.sides for w in side.streamed_weights()]

    def forward_normed_terms(self, x, batch, cache):
        return tuple((side.forward(x, batch, view), scale, w)
                     for side, view, scale, w in zip(self.sides, cache.children, self.scales, self.side_weights))

    def forward_terms(self, x, batch, cache):
        terms = self.forward_normed_terms(x, batch, cache)
        if self.side_eps is None:
            return tuple((t, c) for t, c, _ in terms)
        normed = []
        for t, c, w in terms:       # the sides' norms as launches of their own, for blocks that do not fuse them
            out = self.new(*t.shape)
            ops.rmsnorm(out, t, w, self.side_eps)
            normed.append((out, c))
        return tuple(normed)

    def forward(self, x, batch, cache):
        (a, ca), (b, cb) = self.forward_terms(x, batch, cache)
        out = self.new(*a.shape)
        ops.scaled_sum(out, a, b, ca, cb)
        return out


MIXERS.register("parallel_mixers", ParallelMixers)
