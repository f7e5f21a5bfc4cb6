"""Input filters: what a sub-block's input passes between the norm and the sub-block.

``causal_filter_add``: y_t = x_t + sum_j f[:, j] * x_(t - K + 1 + j), a short causal filter over time on every channel
(no bias, no activation) added to its own input; inputs before a request's first token are zero.  Parameters:
``width``, ``taps`` (K), ``source`` (the checkpoint's name of the filter [width, K]; its last column multiplies the
current token).  Per request it keeps the last K - 1 inputs in float32.  Two such filters over the same input
(``forward_pair``) run in one kernel and share that state.
"""
from __future__ import annotations

from ..kernels import ops
from .base import FILTERS, FixedStateNeed, InputFilter
from .spec import ParamDecl, Source


class CausalFilterAdd(InputFilter):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.width = int(spec["width"])
        self.taps = int(spec["taps"])
        self.source = spec.get("source", "weight")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"a causal filter has 1 to 8 taps, not {self.taps}")

    def params(self):
        # the tensor carries the checkpoint's name, so that a norm and two filters can share a layer's prefix
        return [ParamDecl(self.source, (self.width, self.taps), init="filter_taps",
                          sources=(Source(self.source, 0, self.width),))]

    def bind(self, tensors):
        self.w_weight = tensors[self.source]

    def state_need(self):
        return FixedStateNeed(((self.taps - 1) * self.width,)) if self.taps > 1 else None

    def forward(self, x, batch, state):
        out = self.new(*x.shape)
        ops.causal_filter_add(out, None, x, self.w_weight, None, state, batch)
        return out

    def forward_pair(self, other: "CausalFilterAdd", x, batch, state):
        """(self's output, other's output) over the same x, with the one state they share."""
        a, b = self.new(*x.shape), self.new(*x.shape)
        ops.causal_filter_add(a, b, x, self.w_weight, other.w_weight, state, batch)
        return a, b


FILTERS.register("causal_filter_add", CausalFilterAdd)
