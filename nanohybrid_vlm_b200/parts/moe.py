"""Mixture-of-experts feed-forward with a grouped, bias-corrected softmax router, identity experts and a gated shared
expert; and the clamped gated unit that its experts are made of, as a dense feed-forward of its own.

``clamped_glu`` (dense).  Parameters: ``intermediate_size``, ``limit``, ``alpha`` (default 1.702), ``names`` (the
checkpoint's names of the three matrices; default ("gate", "up", "down")).  g = min(gate(x), limit), u = clamp(up(x),
-limit, limit); down(g * sigmoid(alpha g) * (u + 1)).  Tensors: ``gate_up`` [2 I, width], ``down`` [width, I]; no biases.

``routed_moe``.  Parameters: ``experts`` (E), ``identity`` (I0: the last I0 of the router's E + I0 outputs are experts
whose output is their input; they own no tensors), ``top``, ``groups`` / ``keep`` (the router's outputs, identity ones
included, form ``groups`` equal groups of neighbours and only the ``keep`` best groups can be chosen from; a group's
score is its largest choice score), ``correction`` (True: a learned vector ``correction`` is added to the scores for
the choice only), ``intermediate_size`` / ``limit`` / ``alpha`` (of every expert, a clamped gated unit), ``shared`` (a
PartSpec of a feed-forward that every token passes, its tensors under ``shared.``; None: none), ``shared_gate`` (True:
the shared output is multiplied by sigmoid(sg(x)), one number per token, ``shared.sg`` [1, width]), ``scores``
("softmax", the default, or "sigmoid": each output's score is the sigmoid of its own logit), ``renorm`` (True: the chosen
scores are divided by their sum; False: they are the weights as they are), ``weight_on`` ("output", the default: a
chosen expert's output is multiplied by its weight; "input": its input is, out = sum of expert(w * x)), ``limit`` None
(no clamp) and ``up_shift`` (what is added to the up half, 1 unless given): limit None, alpha 1, up_shift 0 make the
experts plain gated units, down(silu(gate x) * (up x)).

Router: z = router(x) with 32-bit sums; s = softmax(z) over all outputs; choice by s + correction; the weights of the
chosen are their s divided by the sum of the chosen s (+ 1e-20).  The output is the weighted sum of the chosen experts'
outputs, plus the shared term.

Tensors: ``router`` [E + I0 (+ 1), width] (the shared gate's row packed behind the router's, so that one product gives
both), ``correction`` [E + I0] (float32), ``gate`` / ``up`` [E, I, width] and ``down`` [E, width, I] stacked from the
checkpoint's ``e<j>.gate``, ``e<j>.up``, ``e<j>.down``.

A step orders its (token, choice) slots by expert on the device (no host round trip, so a captured step replays), runs
the experts' two products over that order and sums each token's choices in 32-bit.
"""
from __future__ import annotations

from dataclasses import replace

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, FeedForward
from .spec import ParamDecl, Source


class ClampedGLU(FeedForward):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.inter = int(spec["intermediate_size"])
        self.limit = float(spec["limit"])
        self.alpha = float(spec.get("alpha", 1.702))
        self.names = tuple(spec.get("names", ("gate", "up", "down")))

    def params(self):
        H, I = self.env.hidden_size, self.inter
        gate, up, down = self.names
        return [ParamDecl("gate_up", (2 * I, H), sources=(Source(gate, 0, I), Source(up, I, I))),
                ParamDecl("down", (H, I), sources=(Source(down, 0, H),))]

    def streamed_weights(self):
        return [(self.w_gate_up, 0), (self.w_down, 0)]

    def forward(self, x, batch):
        T = x.shape[0]
        gate_up = self.new(T, 2 * self.inter)
        ops.linear(gate_up, x, self.w_gate_up)
        act = self.new(T, self.inter)
        ops.clamped_glu(act, gate_up, self.limit, self.alpha)
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, act, self.w_down)
        return y


class RoutedMoE(FeedForward):
    SHARED_PREFIX = "shared."

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.E = int(spec["experts"])
        self.I0 = int(spec.get("identity", 0))
        self.top = int(spec["top"])
        self.groups = int(spec.get("groups", 1))
        self.keep = int(spec.get("keep", self.groups))
        self.N = self.E + self.I0
        self.inter = int(spec["intermediate_size"])
        limit = spec.get("limit")
        self.limit = float("inf") if limit is None else float(limit)
        self.alpha = float(spec.get("alpha", 1.702))
        self.up_shift = float(spec.get("up_shift", 1.0))
        self.scores = spec.get("scores", "softmax")
        self.renorm = bool(spec.get("renorm", True))
        self.weight_on = spec.get("weight_on", "output")
        if self.scores not in ("softmax", "sigmoid") or self.weight_on not in ("output", "input"):
            raise ValueError(f"unknown router scores {self.scores!r} or weight_on {self.weight_on!r}")
        if self.weight_on == "input" and self.I0:
            raise ValueError("identity experts are not offered with weights on the experts' inputs")
        self.has_correction = bool(spec.get("correction", True))
        if self.E <= 0 or self.I0 < 0 or not 0 < self.top <= self.N:
            raise ValueError(f"{self.E} experts, {self.I0} identity experts, top {self.top}: not a router")
        if self.groups <= 0 or self.N % self.groups or not 0 < self.keep <= self.groups:
            raise ValueError(f"{self.N} router outputs do not form {self.groups} equal groups of which {self.keep} are kept")
        if self.keep * (self.N // self.groups) < self.top:
            raise ValueError(f"the {self.keep} kept groups hold fewer than top = {self.top} outputs")
        shared = spec.get("shared")
        self.shared = FEED_FORWARDS.get(shared.kind)(shared, env) if shared is not None else None
        self.shared_gate = bool(spec.get("shared_gate", False)) and self.shared is not None

    def params(self):
        W, E, I = self.env.hidden_size, self.E, self.inter
        router = [Source("router", 0, self.N)]
        if self.shared_gate:
            router.append(Source(self.SHARED_PREFIX + "sg", self.N, 1))
        decls = [ParamDecl("router", (self.N + int(self.shared_gate), W), sources=tuple(router))]
        if self.has_correction:
            decls.append(ParamDecl("correction", (self.N,), init="zeros_noise", storage="float32"))
        decls += [
            ParamDecl("gate", (E, I, W), sources=tuple(Source(f"e{j}.gate", j, 1, squeeze=True) for j in range(E))),
            ParamDecl("up", (E, I, W), sources=tuple(Source(f"e{j}.up", j, 1, squeeze=True) for j in range(E))),
            ParamDecl("down", (E, W, I), sources=tuple(Source(f"e{j}.down", j, 1, squeeze=True) for j in range(E))),
        ]
        if self.shared is not None:
            for d in self.shared.params():
                srcs = tuple(replace(s, name=self.SHARED_PREFIX + s.name) for s in d.resolved_sources())
                decls.append(replace(d, name=self.SHARED_PREFIX + d.name, sources=srcs))
        return decls

    def bind(self, tensors):
        p = self.SHARED_PREFIX
        super().bind({n: t for n, t in tensors.items() if not n.startswith(p)})
        if self.shared is not None:
            self.shared.bind({n[len(p):]: t for n, t in tensors.items() if n.startswith(p)})

    def streamed_weights(self):
        return self.shared.streamed_weights() if self.shared is not None else []

    def forward(self, x, batch):
        T, W = x.shape
        logits = self.new(T, self.N + int(self.shared_gate), dtype=torch.float32)
        ops.linear_f32(logits, x, self.w_router)
        ids = self.new(T, self.top, dtype=torch.int32)
        weights = self.new(T, self.top, dtype=torch.float32)
        ops.moe_route(ids, weights, logits, self.w_correction if self.has_correction else None, self.N, self.groups, self.keep,
                      scores=self.scores, renorm=self.renorm)
        on_input = self.weight_on == "input"
        # a weight on an expert's input is a factor on the 32-bit sums of its two first products
        y, slot_pos = ops.moe_experts(x, self.w_gate, self.w_up, self.w_down, ids, self.limit, self.alpha, self.up_shift,
                                      weights if on_input else None)
        shared = self.shared.forward(x, batch) if self.shared is not None else None
        out = self.new(T, W)
        ops.moe_combine(out, y, x, ids, None if on_input else weights, slot_pos, self.E, shared,
                        logits[:, self.N] if self.shared_gate else None)
        return out


FEED_FORWARDS.register("clamped_glu", ClampedGLU)
FEED_FORWARDS.register("routed_moe", RoutedMoE)
