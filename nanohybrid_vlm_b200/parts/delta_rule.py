"""The delta rule mixers: the gated delta rule, and the generalised delta rule (class :class:`GeneralDeltaRule` below).

Parameters: ``num_heads`` (value heads H), ``num_qk_heads`` (G: value head h uses q/k head h // (H / G)),
``head_dim`` (d of q and k), ``v_head_dim`` (dv), ``conv`` (taps), ``eps`` (of the output norm).

q, k [G d] and v [H dv] each pass a causal convolution per channel (no bias) and SiLU; q and k become unit vectors
per head (x / sqrt(sum x^2 + 1e-6)), q also times d^-1/2.  beta = sigmoid(b(x)), one per head;
g = exp(-exp(A_log) softplus(a(x) + dt_bias)).  Per head, S [d, dv]: S <- g S; u = beta (v - S^T k);
S <- S + k u^T; o = S^T q (the read-out sees the current token's write).  Each head's o is divided by its root mean
square over dv, multiplied by the weight ``norm`` [dv] (shared by the heads) and by silu(gate(x)); then the output
projection.

Tensors: ``qkvg`` [2 G d + 2 H dv, width] packed from the checkpoint's ``q``, ``k``, ``v``, ``g``; ``ba`` [2 H, width]
from ``b``, ``a``; ``conv`` [2 G d + H dv, taps] from ``q.conv``, ``k.conv``, ``v.conv``; ``A_log``, ``dt_bias`` [H]
(float32); ``norm`` [dv]; ``o`` [width, H dv].  Per request the mixer keeps the convolutions' last taps - 1 inputs and
S, both in float32.  The convolutions write float32, so q, k and v enter the recurrence unrounded; beta, the decay,
the unit vectors, the recurrence and the output norm are 32-bit.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import MIXERS, CompositeNeed, FixedStateNeed, Mixer
from .spec import ParamDecl, Source


class GatedDeltaRule(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.H = int(spec["num_heads"])
        self.G = int(spec.get("num_qk_heads") or self.H)
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("v_head_dim") or self.d)
        self.taps = int(spec["conv"])
        self.eps = float(spec["eps"])
        if self.H % self.G:
            raise ValueError(f"{self.H} heads do not divide into {self.G} q/k heads")
        self.qk_size, self.v_size = self.G * self.d, self.H * self.dv
        self.conv_channels = 2 * self.qk_size + self.v_size

    def params(self):
        W = self.env.hidden_size
        qk, v, C = self.qk_size, self.v_size, self.conv_channels
        return [
            ParamDecl("qkvg", (C + v, W), sources=(Source("q", 0, qk), Source("k", qk, qk), Source("v", 2 * qk, v),
                                                    Source("g", C, v))),
            ParamDecl("ba", (2 * self.H, W), sources=(Source("b", 0, self.H), Source("a", self.H, self.H))),
            ParamDecl("conv", (C, self.taps), sources=(Source("q.conv", 0, qk), Source("k.conv", qk, qk),
                                                       Source("v.conv", 2 * qk, v))),
            ParamDecl("A_log", (self.H,), init="zeros_noise", storage="float32"),
            ParamDecl("dt_bias", (self.H,), init="zeros_noise", storage="float32"),
            ParamDecl("norm", (self.dv,), init="norm"),
            ParamDecl("o", (W, v)),
        ]

    def cache_need(self):
        return CompositeNeed((FixedStateNeed(((self.taps - 1) * self.conv_channels,)),
                              FixedStateNeed((self.H * self.dv * self.d,))))

    def streamed_weights(self):
        return [(self.w_qkvg, 0), (self.w_o, 0)]

    def forward(self, x, batch, cache):
        T = x.shape[0]
        C = self.conv_channels
        conv_state, rule_state = cache.children[0].state, cache.children[1].state
        proj = self.new(T, C + self.v_size)
        ops.linear(proj, x, self.w_qkvg)
        ba = self.new(T, 2 * self.H, dtype=torch.float32)
        ops.linear_f32(ba, x, self.w_ba)
        qkv = self.new(T, C, dtype=torch.float32)      # what enters the recurrence stays 32-bit
        ops.short_conv_silu(qkv, proj[:, :C], self.w_conv, None, conv_state, batch)
        o = self.new(T, self.v_size, dtype=torch.float32)
        ops.delta_rule(o, qkv, ba, self.w_A_log, self.w_dt_bias, rule_state, batch, self.G, self.H, self.d, self.dv)
        gated = self.new(T, self.v_size)
        ops.gated_rmsnorm(gated, o, proj[:, C:], self.w_norm, self.H, self.eps, gate_first=False)
        out = self.new(T, self.env.hidden_size)
        ops.linear(out, gated, self.w_o)
        return out


class GeneralDeltaRule(Mixer):
    """The generalised delta rule: a state per head that decays per key channel and forgets along the unit key at a
    learned rate per key channel.

    Parameters: ``num_heads`` (H), ``head_dim`` (d of r, k and v alike), ``decay_rank`` (the inner size of the decay's
    two-step projection), ``decay_floor`` (the decay is exp(-decay_floor * sigmoid(.)), so it stays above
    exp(-decay_floor); default exp(-1/2)), ``eps`` (of the output norm).

    r, k, v = three projections of the input, [H d] each.  Per head and key channel: the decay
    w = exp(-decay_floor * sigmoid(w2 tanh(w1 x) + w0)) and the removal rate a = sigmoid(a x + a.b).  With the unit key
    u = k / sqrt(sum k^2 + 1e-6), per head S [d, d]:  S <- diag(w) S - (a * u) (u^T S) + k v^T, both the decay and the
    removal reading the state of the token before; o = S^T r sees the current token's write.  Each head's o is divided by
    its root mean square, multiplied by the weight ``norm`` [H d] and by sigmoid(g x); then the output projection.

    Tensors: ``rkvg`` [4 H d, width] packed from the checkpoint's ``r``, ``k``, ``v``, ``g``; ``aw1`` [H d + rank, width]
    from ``a``, ``w1``; ``a.b``, ``w0``, ``norm`` [H d]; ``w2`` [H d, rank]; ``o`` [width, H d].  Per request the mixer
    keeps S in float32.  The two small projections give float32 sums; tanh, sigmoid, the exponentials, the unit key, the
    recurrence and the output norm are 32-bit."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.H = int(spec["num_heads"])
        self.d = int(spec["head_dim"])
        self.rank = int(spec["decay_rank"])
        self.eps = float(spec["eps"])
        self.decay_floor = float(spec.get("decay_floor", math.exp(-0.5)))
        if min(self.H, self.d, self.rank) <= 0:
            raise ValueError("the generalised delta rule: heads, head_dim and decay_rank must be positive")
        self.n = self.H * self.d

    def params(self):
        W, n = self.env.hidden_size, self.n
        return [
            ParamDecl("rkvg", (4 * n, W), sources=(Source("r", 0, n), Source("k", n, n), Source("v", 2 * n, n),
                                                   Source("g", 3 * n, n))),
            ParamDecl("aw1", (n + self.rank, W), sources=(Source("a", 0, n), Source("w1", n, self.rank))),
            ParamDecl("a.b", (n,), init="gate_bias"),
            ParamDecl("w0", (n,), init="gate_bias"),
            ParamDecl("w2", (n, self.rank), init="unit"),
            ParamDecl("norm", (n,), init="norm"),
            ParamDecl("o", (W, n)),
        ]

    def cache_need(self):
        return FixedStateNeed((self.H * self.d * self.d,))

    def streamed_weights(self):
        return [(self.w_rkvg, 0), (self.w_o, 0)]

    def forward(self, x, batch, cache):
        T, n = x.shape[0], self.n
        proj = self.new(T, 4 * n)
        ops.linear(proj, x, self.w_rkvg)
        aw = self.new(T, n + self.rank, dtype=torch.float32)
        ops.linear_f32(aw, x, self.w_aw1)
        o = self.new(T, n, dtype=torch.float32)
        ops.general_delta(o, proj, aw, self.w_a_b, self.w_w2, self.w_w0, cache.state, batch, self.H, self.d,
                          self.decay_floor)
        gated = self.new(T, n)
        ops.gated_rmsnorm(gated, o, proj[:, 3 * n:], self.w_norm, self.H, self.eps, gate_first=False, gate="sigmoid")
        out = self.new(T, self.env.hidden_size)
        ops.linear(out, gated, self.w_o)
        return out


MIXERS.register("gated_delta_rule", GatedDeltaRule)
MIXERS.register("general_delta_rule", GeneralDeltaRule)
